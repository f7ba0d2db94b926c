"""Host half of the bucket-width search: the cost model on per-class statistics.

The reference keeps, per bucket, a Python list of row ids and a Python set of column ids
(format_matrix_market.py:12-37) although the cost model only ever reads their lengths
(format_algos.py:1078, 1082).  The device pass (``lf_hyb_stats``) delivers exactly those
lengths: three counters per (partition, width class) and, per partition, a 2048-bin
histogram over the per-column bitmask of classes that touch the column.  A merged bucket is
a set of classes; its number of distinct columns is the sum of the bins whose mask
intersects that set.

Everything order- or rounding-sensitive is kept as the reference has it:
  * a bucket that is created by a move lands at the END of the dict, and costs are summed
    in dict order (format_algos.py:637-648, 1058-1095);
  * the single-row fix-up walks a descending SNAPSHOT of the widths (format_algos.py:940-953)
    and a lone width-1 row is moved up to the next width of that snapshot, adding
    ``1 // width == 0`` rows (format_algos.py:903-923);
  * the cost is computed with Python ints and true division (format_algos.py:1084-1087) and a
    candidate wins only when strictly cheaper (format_algos.py:768).
"""
from __future__ import annotations

from typing import Dict, List

import numpy as np

NUM_CLASSES = 11
BINS = 1 << NUM_CLASSES


class _Bucket:
    __slots__ = ("num_rows", "nnz", "n_row_ids", "classes")

    def __init__(self, num_rows: int, nnz: int, n_row_ids: int, classes: int):
        self.num_rows = num_rows      # cost-model row estimate
        self.nnz = nnz
        self.n_row_ids = n_row_ids    # len(Bucket.row_indices)
        self.classes = classes        # bitmask of width classes merged into this bucket


def _move(pool: Dict[int, _Bucket], src_w: int, dst_w: int) -> None:
    src = pool[src_w]
    extra = src.num_rows * (src_w // dst_w)
    if dst_w in pool:
        dst = pool[dst_w]
        dst.num_rows += extra
        dst.nnz += src.nnz
        dst.n_row_ids += src.n_row_ids
        dst.classes |= src.classes
    else:
        pool[dst_w] = _Bucket(extra, src.nnz, src.n_row_ids, src.classes)
    del pool[src_w]


class _ColumnCounter:
    """len(col_indices) of a merged bucket from the class-mask histogram of one partition."""

    def __init__(self, hist_row: np.ndarray):
        self._hist = np.asarray(hist_row, dtype=np.int64)
        self._bins = np.arange(BINS, dtype=np.int64)
        self._memo: Dict[int, int] = {}

    def __call__(self, classes: int) -> int:
        got = self._memo.get(classes)
        if got is None:
            got = int(self._hist[(self._bins & classes) != 0].sum())
            self._memo[classes] = got
        return got


def _cost(pool: Dict[int, _Bucket], ncols: _ColumnCounter, feat_size: int, num_parts: int):
    wmax = max(pool.keys())
    total = 0
    for w, b in pool.items():
        per_block = wmax // w
        padded = ((b.num_rows + per_block - 1) // per_block) * per_block
        c_index = 2 * padded * w
        c_gather = ncols(b.classes) * feat_size
        atomic = num_parts > 1 or w == wmax
        weight = padded / b.n_row_ids if atomic else 1
        c_out = weight * b.n_row_ids * feat_size
        total += c_index + c_gather + c_out
    return total


def _fix_single_row_buckets(pool: Dict[int, _Bucket]) -> None:
    snapshot = sorted(pool.keys(), reverse=True)
    for w in snapshot:
        if pool[w].num_rows != 1:
            continue
        if w > 1:
            _move(pool, w, w // 2)
            continue
        target, top = 2, max(snapshot)
        while target <= top and target not in snapshot:
            target *= 2
        if target > top:
            raise ValueError("The partition is too small, only having 1 non-zero element.")
        _move(pool, 1, target)


def _choose(pool: Dict[int, _Bucket], ncols: _ColumnCounter, feat_size: int, num_parts: int,
            cost_out: list = None) -> List[int]:
    best_cost = _cost(pool, ncols, feat_size, num_parts)
    best = sorted(pool.keys())
    cur = max(pool.keys())
    nxt = cur // 2
    while nxt >= 1:
        _move(pool, cur, nxt)
        c = _cost(pool, ncols, feat_size, num_parts)
        if c < best_cost:
            best, best_cost = sorted(pool.keys()), c
        cur, nxt = nxt, nxt // 2
    if cost_out is not None:
        cost_out.append(best_cost)
    return best


def search_from_stats(class_stats: np.ndarray, colmask_hist: np.ndarray, feat_size: int,
                      num_parts: int, cost_out: list = None) -> List[List[int]]:
    """``class_stats``: int64[P, 11, 3] = (num_rows, nnz, #rows); ``colmask_hist``: int64[P, 2048].
    ``cost_out`` (a list) receives the winning cost of every non-empty partition."""
    class_stats = np.asarray(class_stats, dtype=np.int64).reshape(num_parts, NUM_CLASSES, 3)
    colmask_hist = np.asarray(colmask_hist, dtype=np.int64).reshape(num_parts, BINS)
    pools: List[Dict[int, _Bucket]] = []
    for p in range(num_parts):
        pool: Dict[int, _Bucket] = {}
        for k in range(NUM_CLASSES):
            num_rows, nnz, n_ids = (int(x) for x in class_stats[p, k])
            if n_ids:
                pool[1 << k] = _Bucket(num_rows, nnz, n_ids, 1 << k)
        pools.append(pool)
    # the fix-up pass visits every partition before any width is chosen (format_algos.py:1021,
    # 1030), so a partition with a single nonzero raises even if it is not the first one
    for pool in pools:
        _fix_single_row_buckets(pool)
    out: List[List[int]] = []
    for p, pool in enumerate(pools):
        out.append(_choose(pool, _ColumnCounter(colmask_hist[p]), feat_size, num_parts, cost_out) if pool else [])
    return out
