"""Seeded synthetic matrices standing in for the reference's GNN graphs and SuiteSparse files.

The reference benchmarks on seven downloaded graphs (proc05.spmm.end-to-end.py:22) that
are not available offline.  The five generators below produce the matrices the benchmark
configurations describe, on the host with ``numpy.random.default_rng(seed)`` so that every
machine sees identical CSR arrays: ``int32`` indices, columns sorted inside a row, and no
duplicate ``(row, col)`` pair (duplicates make the reference's bucketing inconsistent:
degrees are counted on COO entries, format_algos.py:249-252, entries are taken from the
merged CSR, format_algos.py:254).

Each generator takes the full-size dimension by default and a smaller ``M`` for tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Tuple

import numpy as np


@dataclass
class Csr:
    indptr: np.ndarray      # int64[M + 1]
    indices: np.ndarray     # int32[nnz], sorted inside each row, distinct
    data: np.ndarray        # float32[nnz]
    shape: Tuple[int, int]
    name: str = "synthetic"

    @property
    def nnz(self) -> int:
        return int(self.indptr[-1])

    def tocoo(self):
        import scipy.sparse as sp
        rows = np.repeat(np.arange(self.shape[0], dtype=np.int32), np.diff(self.indptr))
        return sp.coo_matrix((self.data, (rows, self.indices)), shape=self.shape)

    def toscipy(self):
        import scipy.sparse as sp
        return sp.csr_matrix((self.data, self.indices, self.indptr), shape=self.shape)


def _sorted_unique(a: np.ndarray) -> np.ndarray:
    """``np.unique(a)`` for an integer array by sort + neighbour compare (sorts ``a`` in place)."""
    a.sort()
    if a.size == 0:
        return a
    keep = np.ones(a.size, dtype=bool)
    np.not_equal(a[1:], a[:-1], out=keep[1:])
    return a[keep]


def _merge_unique(keys: np.ndarray, new: np.ndarray) -> np.ndarray:
    """``np.unique(np.concatenate([keys, new]))`` when ``keys`` is already sorted and distinct and
    ``new`` is much shorter: insert instead of sorting everything again."""
    new = _sorted_unique(new)
    if keys.size == 0:
        return new
    pos = np.searchsorted(keys, new)
    dup = keys[np.minimum(pos, keys.size - 1)] == new
    return np.insert(keys, pos[~dup], new[~dup])


def _distinct_uniform_columns(rng, lens: np.ndarray, K: int):
    """For every row r draw ``lens[r]`` distinct uniform columns; returns flat sorted keys
    ``row * K + col`` (so rows come out contiguous and columns ascending)."""
    M = len(lens)
    lens = np.asarray(lens, dtype=np.int64)
    need = lens.copy()
    # rows that want a large share of all columns: rejection would crawl, cut a permutation
    dense = np.nonzero(lens * 4 > K)[0]
    dense_keys = [r * K + np.sort(rng.permutation(K)[:lens[r]]).astype(np.int64) for r in dense]
    keys = np.concatenate(dense_keys) if dense_keys else np.empty(0, dtype=np.int64)
    need[dense] = 0
    while True:
        total = int(need.sum())
        if total == 0:
            break
        r = np.repeat(np.arange(M, dtype=np.int64), need)
        c = rng.integers(0, K, size=total, dtype=np.int64)
        keys = _merge_unique(keys, r * K + c) if keys.size else _sorted_unique(r * K + c)
        have = np.bincount(keys // K, minlength=M)
        need = lens - have
    return keys


def _csr_from_keys(keys: np.ndarray, M: int, K: int):
    rows = keys // K
    indices = (keys - rows * K).astype(np.int32)
    indptr = np.zeros(M + 1, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=M), out=indptr[1:])
    return indptr, indices


def dense_features(K: int, N: int, seed: int) -> np.ndarray:
    """B ~ N(0, 1) float32, row-major ``[K, N]``."""
    return np.random.default_rng(seed + 1).standard_normal((K, N), dtype=np.float32)


def zipf_rows(M: int = 16384, seed: int = 0, mean: float = 16.0, cap: int = 2048) -> Csr:
    """Config 1: Zipf(1.8) row lengths clipped to [1, cap], rescaled to ``mean`` nnz/row."""
    rng = np.random.default_rng(seed)
    cap = min(cap, M)
    raw = np.clip(rng.zipf(1.8, M), 1, cap).astype(np.float64)
    lens = np.clip(np.rint(raw * (mean / raw.mean())), 1, cap).astype(np.int64)
    keys = _distinct_uniform_columns(rng, lens, M)
    indptr, indices = _csr_from_keys(keys, M, M)
    data = rng.uniform(-1.0, 1.0, size=len(indices)).astype(np.float32)
    return Csr(indptr, indices, data, (M, M), f"zipf_{M}")


def power_law_graph(M: int = 1 << 20, seed: int = 1, mean: float = 14.0, cap: int = 50_000,
                    exponent: float = 2.1) -> Csr:
    """Config 2: power-law out-degrees, degree-proportional (preferential) column choice,
    unweighted adjacency then row-normalised."""
    rng = np.random.default_rng(seed)
    cap = min(cap, M)
    raw = (1.0 - rng.random(M)) ** (-1.0 / (exponent - 1.0))
    scale = 1.0
    for _ in range(8):  # clipping changes the mean; re-scale until it settles
        deg = np.clip(np.rint(raw * scale), 1, cap)
        scale *= mean / deg.mean()
    deg = np.clip(np.rint(raw * scale), 1, cap).astype(np.int64)
    weight = np.cumsum((deg + 1).astype(np.float64))
    total = int(deg.sum())
    r = np.repeat(np.arange(M, dtype=np.int64), deg)
    c = np.searchsorted(weight, rng.random(total) * weight[-1], side="right").astype(np.int64)
    np.minimum(c, M - 1, out=c)
    keys = _sorted_unique(r * M + c)       # in-row duplicates dropped
    indptr, indices = _csr_from_keys(keys, M, M)
    lens = np.diff(indptr)
    data = np.repeat((1.0 / np.maximum(lens, 1)).astype(np.float32), lens)
    return Csr(indptr, indices, data, (M, M), f"powerlaw_{M}")


def uniform_rows(M: int = 1 << 22, seed: int = 2, per_row: int = 32) -> Csr:
    """Config 3: exactly ``per_row`` distinct uniform columns in every row."""
    rng = np.random.default_rng(seed)
    cols = rng.integers(0, M, size=(M, per_row), dtype=np.int32)
    while True:
        cols.sort(axis=1)
        bad = np.nonzero((cols[:, 1:] == cols[:, :-1]).any(axis=1))[0]
        if len(bad) == 0:
            break
        cols[bad] = rng.integers(0, M, size=(len(bad), per_row), dtype=np.int32)
    indptr = np.arange(M + 1, dtype=np.int64) * per_row
    data = rng.uniform(-1.0, 1.0, size=M * per_row).astype(np.float32)
    return Csr(indptr, cols.reshape(-1), data, (M, M), f"uniform{per_row}_{M}")


def skewed_rows(M: int = 1 << 20, seed: int = 3, heavy_rows: int = 64, heavy_len: int = 100_000) -> Csr:
    """Config 4: a few very long rows, the rest log-normal(2, 1.2) lengths."""
    rng = np.random.default_rng(seed)
    heavy_len = min(heavy_len, M // 8)
    lens = np.clip(np.rint(rng.lognormal(2.0, 1.2, M)), 1, M).astype(np.int64)
    heavy = rng.choice(M, size=min(heavy_rows, M), replace=False)
    lens[heavy] = heavy_len
    keys = _distinct_uniform_columns(rng, lens, M)
    indptr, indices = _csr_from_keys(keys, M, M)
    data = rng.uniform(-1.0, 1.0, size=len(indices)).astype(np.float32)
    return Csr(indptr, indices, data, (M, M), f"skew_{M}")


def banded_blocks(M: int = 1 << 21, seed: int = 4, block: int = 8, per_block_row: int = 8,
                  half_band: int = 4096):
    """Config 5: dense ``block x block`` tiles on a banded pattern.

    Returns ``(bsr_indptr int32[Mb+1], bsr_indices int32[nb], blocks float32[nb, block, block])``
    with block columns sorted inside a block row; the diagonal block is always present.
    """
    rng = np.random.default_rng(seed)
    Mb = M // block
    half_band = min(half_band, max(1, Mb // 2))
    bi = np.arange(Mb, dtype=np.int64)
    lo = np.maximum(bi - half_band, 0)
    hi = np.minimum(bi + half_band, Mb - 1)
    span = hi - lo + 1
    per_block_row = int(min(per_block_row, span.min()))
    cols = np.empty((Mb, per_block_row), dtype=np.int64)
    cols[:, 0] = bi
    todo = np.arange(Mb)
    cols[:, 1:] = lo[:, None] + (rng.random((Mb, per_block_row - 1)) * span[:, None]).astype(np.int64)
    while True:
        cols.sort(axis=1)
        bad = todo[(cols[:, 1:] == cols[:, :-1]).any(axis=1)]
        if len(bad) == 0:
            break
        cols[bad, 0] = bad
        cols[bad, 1:] = lo[bad, None] + (rng.random((len(bad), per_block_row - 1)) * span[bad, None]).astype(np.int64)
    indptr = (np.arange(Mb + 1, dtype=np.int64) * per_block_row).astype(np.int32)
    nb = Mb * per_block_row
    blocks = rng.uniform(-1.0, 1.0, size=(nb, block, block)).astype(np.float32)
    return indptr, cols.reshape(-1).astype(np.int32), blocks, (M, M)


def bsr_to_csr(bsr_indptr, bsr_indices, blocks, shape) -> Csr:
    """Expand a BSR matrix to element CSR (sorted columns)."""
    nb, R, C = blocks.shape
    Mb = len(bsr_indptr) - 1
    per_row = np.diff(bsr_indptr).astype(np.int64)
    # element row r of block row I holds, for each block of I in order, C consecutive columns
    elem_per_row = np.repeat(per_row * C, R)
    indptr = np.zeros(Mb * R + 1, dtype=np.int64)
    np.cumsum(elem_per_row, out=indptr[1:])
    blk_of_row = np.repeat(np.arange(Mb), per_row)               # block -> block row
    pos_in_row = np.arange(nb) - np.repeat(bsr_indptr[:-1].astype(np.int64), per_row)
    indices = np.empty(int(indptr[-1]), dtype=np.int32)
    data = np.empty(int(indptr[-1]), dtype=np.float32)
    for r in range(R):
        base = indptr[blk_of_row * R + r] + pos_in_row * C       # start of this block in row r
        for c in range(C):
            indices[base + c] = bsr_indices.astype(np.int64) * C + c
            data[base + c] = blocks[:, r, c]
    return Csr(indptr, indices, data, tuple(shape), "banded_blocks")
