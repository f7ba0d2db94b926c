"""TEST INFRASTRUCTURE ONLY -- CPU restatement of LiteForm's composed-format (hyb/CELL) path.

This file restates, in NumPy, what the reference's pure-Python code computes, so that
the CUDA library can be checked against it on machines where the reference checkout is
not present.  It is never imported by the shipped package; only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may call it.

Parity status: *pinned* for the format side.  ``tests/test_oracle_vs_reference.py``
runs the unmodified reference (loaded by ``reference_shim.py``) against every function
below on seeded inputs, and ``tests/golden/`` holds digests of the reference's own
output that the oracle must reproduce on any machine.  The SpMM product has no golden
vectors in the reference (its only check, format_algos.py:596-597, compares against
SciPy and is switched off); the product oracle is therefore SciPy itself, which is
exactly what the reference's ``MTX.dot`` (format_matrix_market.py:89-99) calls.

Reference functions restated here (paths inside the reference project):
  * ``get_init_buckets``            playground_pipline/format_algos.py:819-900
  * ``move_largest_bucket``         playground_pipline/format_algos.py:623-648
  * ``move_width_one_bucket``       playground_pipline/format_algos.py:903-923
  * ``modify_single_row_buckets``   playground_pipline/format_algos.py:928-953
  * ``get_memory_cost``             playground_pipline/format_algos.py:1035-1166
  * ``modify_bucket_widths``        playground_pipline/format_algos.py:709-774
  * ``get_bucket_config``           playground_pipline/format_algos.py:777-816
  * ``search_bucket_config``        playground_pipline/format_algos.py:988-1032
  * ``build_hyb_format``            playground_pipline/format_algos.py:226-385
  * ``MTX.dot``                     playground_pipline/format_matrix_market.py:89-99
"""
from __future__ import annotations

import bisect
import hashlib
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

import numpy as np
import scipy.sparse as sp

WIDTH_LIMIT = 1024  # format_algos.py:821


# --------------------------------------------------------------------------------------
# bucket statistics (get_init_buckets)
# --------------------------------------------------------------------------------------
@dataclass
class BucketStat:
    """What the cost model reads from a reference ``Bucket`` (format_matrix_market.py:12-37)."""
    width: int
    num_rows: int                 # cost-model row estimate (a clipped row counts width//1024 times)
    nnz: int
    row_ids: np.ndarray           # rows that live in the bucket (only the length is used)
    cols: np.ndarray              # sorted distinct columns touched by those rows

    def merged_into(self, other: "BucketStat", extra_rows: int) -> None:
        other.num_rows += extra_rows
        other.nnz += self.nnz
        other.row_ids = np.concatenate([other.row_ids, self.row_ids])
        other.cols = np.union1d(other.cols, self.cols)


def _ceil_log2(deg: np.ndarray) -> np.ndarray:
    """``math.ceil(math.log2(d))`` for positive integers (format_algos.py:875), exactly."""
    d = np.asarray(deg, dtype=np.int64)
    k = np.ceil(np.log2(d.astype(np.float64))).astype(np.int64)
    # integer fix-ups so the result never depends on float rounding
    k += (np.int64(1) << k) < d
    k -= (k > 0) & ((np.int64(1) << np.maximum(k - 1, 0)) >= d)
    return k


def partition_size(num_cols: int, num_parts: int) -> int:
    return (num_cols + num_parts - 1) // num_parts  # format_algos.py:241, 836


def init_buckets(row: np.ndarray, col: np.ndarray, shape: Tuple[int, int], num_parts: int,
                 width_limit: int = WIDTH_LIMIT) -> List[Dict[int, BucketStat]]:
    """Per partition: ``{width: BucketStat}`` sorted by width, from COO entries."""
    M, K = shape
    psz = partition_size(K, num_parts)
    row = np.asarray(row, dtype=np.int64)
    col = np.asarray(col, dtype=np.int64)
    part = col // psz
    out: List[Dict[int, BucketStat]] = []
    for p in range(num_parts):
        sel = part == p
        r_p, c_p = row[sel], col[sel]
        deg = np.bincount(r_p, minlength=M).astype(np.int64)
        live = np.nonzero(deg)[0]
        k = _ceil_log2(deg[live])
        width = np.int64(1) << k
        reps = np.ones(len(live), dtype=np.int64)
        over = width > width_limit
        reps[over] = width[over] // width_limit
        width[over] = width_limit
        row_width = np.zeros(M, dtype=np.int64)
        row_width[live] = width
        pool: Dict[int, BucketStat] = {}
        for w in np.unique(width):
            rows_w = live[width == w]
            pool[int(w)] = BucketStat(
                width=int(w),
                num_rows=int(reps[width == w].sum()),
                nnz=int(deg[rows_w].sum()),
                row_ids=rows_w,
                cols=np.unique(c_p[row_width[r_p] == w]),
            )
        out.append(dict(sorted(pool.items())))
    return out


def bucket_counters(row: np.ndarray, col: np.ndarray, shape: Tuple[int, int], num_parts: int):
    """The bucket statistics of ``init_buckets`` (format_algos.py:819-900) in the counter form the
    CUDA library emits: ``class_stats int64[P, 11, 3]`` = (num_rows, nnz, len(row_indices)) per
    width class ``k`` (width ``2**k``), and ``colmask_hist int64[P, 2048]`` = number of columns of
    the partition whose set of touching classes is the bin's bit pattern (so that the size of the
    union of ``col_indices`` over any set of classes is a sum of bins)."""
    pools = init_buckets(row, col, shape, num_parts)
    K = shape[1]
    psz = partition_size(K, num_parts)
    n_classes = WIDTH_LIMIT.bit_length()          # widths 1 .. 1024
    stats = np.zeros((num_parts, n_classes, 3), dtype=np.int64)
    hist = np.zeros((num_parts, 1 << n_classes), dtype=np.int64)
    for p, pool in enumerate(pools):
        colmask = np.zeros(K, dtype=np.int64)
        for w, b in pool.items():
            k = int(w).bit_length() - 1
            stats[p, k] = (b.num_rows, b.nnz, len(b.row_ids))
            colmask[b.cols] |= np.int64(1) << k
        touched = np.nonzero(colmask)[0]
        assert touched.size == 0 or (touched // psz == p).all()
        np.add.at(hist[p], colmask[touched], 1)
    return stats, hist


# --------------------------------------------------------------------------------------
# the dictionary surgery of the width search
# --------------------------------------------------------------------------------------
def move_bucket(pool: Dict[int, BucketStat], src_w: int, dst_w: int) -> None:
    """Fold bucket ``src_w`` into ``dst_w``; a new key lands at the END of the dict."""
    src = pool[src_w]
    extra = src.num_rows * (src_w // dst_w)
    if dst_w in pool:
        src.merged_into(pool[dst_w], extra)
    else:
        pool[dst_w] = BucketStat(dst_w, extra, src.nnz, src.row_ids, src.cols)
    del pool[src_w]


def fix_single_row_buckets(pools: List[Dict[int, BucketStat]]) -> None:
    for pool in pools:
        snapshot = sorted(pool.keys(), reverse=True)
        for w in snapshot:
            if pool[w].num_rows != 1:
                continue
            if w > 1:
                move_bucket(pool, w, w // 2)
                continue
            # a lone width-1 row goes UP to the next width of the snapshot
            target, top = 2, max(snapshot)
            while target <= top and target not in snapshot:
                target *= 2
            if target > top:
                raise ValueError("The partition is too small, only having 1 non-zero element.")
            move_bucket(pool, 1, target)


def memory_cost(pool: Dict[int, BucketStat], feat_size: int, num_parts: int):
    """The scalar that ranks width sets; same operations, same order, Python numbers."""
    wmax = max(pool.keys())
    total = 0
    for w, b in pool.items():
        per_block = wmax // w
        padded_rows = ((b.num_rows + per_block - 1) // per_block) * per_block
        c_index = 2 * padded_rows * w
        c_gather = len(b.cols) * feat_size
        atomic = num_parts > 1 or w == wmax
        outs = len(b.row_ids)
        weight = padded_rows / outs if atomic else 1
        c_out = weight * outs * feat_size
        total += c_index + c_gather + c_out
    return total


def choose_widths(pool: Dict[int, BucketStat], feat_size: int, num_parts: int) -> List[int]:
    best_cost = memory_cost(pool, feat_size, num_parts)
    best = sorted(pool.keys())
    cur = max(pool.keys())
    nxt = cur // 2
    while nxt >= 1:
        move_bucket(pool, cur, nxt)
        c = memory_cost(pool, feat_size, num_parts)
        if c < best_cost:
            best, best_cost = sorted(pool.keys()), c
        cur, nxt = nxt, nxt // 2
    return best


def search_bucket_config(row, col, shape, num_parts: int, feat_size: int) -> List[List[int]]:
    pools = init_buckets(row, col, shape, num_parts)
    fix_single_row_buckets(pools)
    return [choose_widths(pool, feat_size, num_parts) if pool else [] for pool in pools]


# --------------------------------------------------------------------------------------
# build_hyb_format
# --------------------------------------------------------------------------------------
def build_hyb(indptr, indices, shape, bucket_widths: Sequence[Sequence[int]], data=None,
              row_range=None):
    """Closed form of the builder on a duplicate-free CSR with sorted columns.

    Returns ``(rows, cols, mask, vals)`` nested ``[partition][bucket]``; ``rows[p][b]`` is
    ``int32[R]``, the others ``[R, w]`` (``int32``, ``int32``, ``float32``).  ``vals`` holds
    ``data`` where ``mask == 1`` and 0 elsewhere (``mask`` as float when ``data`` is None,
    which is what the reference uploads as A-values, format_algos.py:568-570).
    ``row_range=(r0, r1)`` restricts the build to those matrix rows (row ids stay global).
    """
    M, K = shape
    P = len(bucket_widths)
    psz = partition_size(K, P)
    indptr = np.asarray(indptr, dtype=np.int64)
    indices = np.asarray(indices, dtype=np.int64)
    r0, r1 = (0, M) if row_range is None else row_range
    lo, hi = indptr[r0], indptr[r1]
    ent_row = np.repeat(np.arange(r0, r1, dtype=np.int64), np.diff(indptr[r0:r1 + 1]))
    ent_col = indices[lo:hi]
    ent_val = None if data is None else np.asarray(data, dtype=np.float32)[lo:hi]
    ent_part = ent_col // psz
    rows_out, cols_out, mask_out, vals_out = [], [], [], []
    for p in range(P):
        W = list(bucket_widths[p])
        rows_p, cols_p, mask_p, vals_p = [], [], [], []
        sel = ent_part == p
        e_row, e_col = ent_row[sel], ent_col[sel]
        e_val = None if ent_val is None else ent_val[sel]
        deg = np.bincount(e_row - r0, minlength=r1 - r0).astype(np.int64)
        if W:
            bucket_of_row = np.minimum(np.searchsorted(np.asarray(W), deg, side="left"), len(W) - 1)
        # position of every entry inside its row's partition segment
        seg_start = np.zeros(r1 - r0 + 1, dtype=np.int64)
        np.cumsum(deg, out=seg_start[1:])
        pos_in_row = np.arange(len(e_row), dtype=np.int64) - seg_start[e_row - r0]
        for b, w in enumerate(W):
            live = np.nonzero((bucket_of_row == b) & (deg > 0))[0]
            n_ell = -(-deg[live] // w)
            first = np.zeros(len(live) + 1, dtype=np.int64)
            np.cumsum(n_ell, out=first[1:])
            R = int(first[-1])
            rr = np.repeat(live + r0, n_ell).astype(np.int32)
            cc = np.zeros(R * w, dtype=np.int32)
            mm = np.zeros(R * w, dtype=np.int32)
            vv = np.zeros(R * w, dtype=np.float32)
            first_of_row = np.full(r1 - r0, -1, dtype=np.int64)
            first_of_row[live] = first[:-1]
            mine = first_of_row[e_row - r0] >= 0
            dst = first_of_row[e_row[mine] - r0] * w + pos_in_row[mine]
            cc[dst] = e_col[mine]
            mm[dst] = 1
            vv[dst] = 1.0 if e_val is None else e_val[mine]
            rows_p.append(rr)
            cols_p.append(cc.reshape(R, w))
            mask_p.append(mm.reshape(R, w))
            vals_p.append(vv.reshape(R, w))
        rows_out.append(rows_p)
        cols_out.append(cols_p)
        mask_out.append(mask_p)
        vals_out.append(vals_p)
    return rows_out, cols_out, mask_out, vals_out


def build_hyb_entrywise(indptr, indices, shape, bucket_widths):
    """Entry-by-entry restatement (the reference's control flow, format_algos.py:268-371).

    Quadratic-free but interpreted: use on small matrices to cross-check ``build_hyb``.
    """
    M, K = shape
    P = len(bucket_widths)
    psz = partition_size(K, P)
    deg = [[0] * M for _ in range(P)]
    for r in range(M):
        for e in range(indptr[r], indptr[r + 1]):
            deg[int(indices[e]) // psz][r] += 1
    rows = [[[] for _ in W] for W in bucket_widths]
    cols = [[[] for _ in W] for W in bucket_widths]
    mask = [[[] for _ in W] for W in bucket_widths]

    def pad(p, b, w):
        fill = (-len(cols[p][b])) % w
        cols[p][b].extend([0] * fill)
        mask[p][b].extend([0] * fill)

    for r in range(M):
        for e in range(indptr[r], indptr[r + 1]):
            c = int(indices[e])
            p = c // psz
            W = bucket_widths[p]
            b = min(bisect.bisect_left(W, deg[p][r]), len(W) - 1)
            w = W[b]
            if len(cols[p][b]) % w == 0:
                rows[p][b].append(r)
            elif rows[p][b][-1] != r:
                pad(p, b, w)
                rows[p][b].append(r)
            cols[p][b].append(c)
            mask[p][b].append(1)
    R_out, C_out, M_out = [], [], []
    for p in range(P):
        rp, cp, mp = [], [], []
        for b, w in enumerate(bucket_widths[p]):
            pad(p, b, w)
            n = len(rows[p][b])
            rp.append(np.asarray(rows[p][b], dtype=np.int32).reshape(n))
            cp.append(np.asarray(cols[p][b], dtype=np.int32).reshape(n, w))
            mp.append(np.asarray(mask[p][b], dtype=np.int32).reshape(n, w))
        R_out.append(rp)
        C_out.append(cp)
        M_out.append(mp)
    return R_out, C_out, M_out


# --------------------------------------------------------------------------------------
# products
# --------------------------------------------------------------------------------------
def spmm_scipy(indptr, indices, data, shape, B: np.ndarray) -> np.ndarray:
    """``A @ B`` the way the reference's ``MTX.dot`` does it: SciPy CSC times dense."""
    A = sp.csr_matrix((np.asarray(data), np.asarray(indices), np.asarray(indptr)), shape=shape)
    return np.asarray(A.tocsc().dot(B))


def spmm_scipy_csr(indptr, indices, data, shape, B: np.ndarray) -> np.ndarray:
    A = sp.csr_matrix((np.asarray(data), np.asarray(indices), np.asarray(indptr)), shape=shape)
    return np.asarray(A.dot(B))


def spmm_prebuilt(A_csr, B: np.ndarray) -> np.ndarray:
    """The same SciPy product on an already constructed matrix (what the CPU baseline times)."""
    return A_csr @ B


def spmm_hyb(rows, cols, vals, num_rows: int, B: np.ndarray) -> np.ndarray:
    """Evaluate ``C[row[i], :] += sum_j vals[i, j] * B[cols[i, j], :]`` over all buckets
    (the arithmetic of the generated kernel, format_algos.py:99-102 with the ELL axes of
    format_algos.py:55-70), in float64."""
    C = np.zeros((num_rows, B.shape[1]), dtype=np.float64)
    B64 = B.astype(np.float64)
    for rows_p, cols_p, vals_p in zip(rows, cols, vals):
        for r, c, v in zip(rows_p, cols_p, vals_p):
            if r.size == 0:
                continue
            w = c.shape[1]
            step = max(1, (1 << 22) // max(1, w * B.shape[1]))
            for s in range(0, len(r), step):
                part = np.einsum("ij,ijk->ik", v[s:s + step].astype(np.float64), B64[c[s:s + step]])
                np.add.at(C, r[s:s + step], part)
    return C


def bsr_from_csr(indptr, indices, data, shape, block: int = 8):
    """Block format oracle: SciPy's own BSR conversion (as format_matrix_market.py:137 uses)."""
    A = sp.csr_matrix((np.asarray(data), np.asarray(indices), np.asarray(indptr)), shape=shape)
    Bm = A.tobsr(blocksize=(block, block))
    Bm.sort_indices()
    return Bm.indptr.astype(np.int32), Bm.indices.astype(np.int32), Bm.data


# --------------------------------------------------------------------------------------
# digests (golden fixtures store these instead of multi-GB arrays)
# --------------------------------------------------------------------------------------
def digest_hyb(bucket_widths, rows, cols, mask) -> str:
    """sha256 over widths and the int32 casts of every array, in (partition, bucket) order."""
    h = hashlib.sha256()
    for p, W in enumerate(bucket_widths):
        h.update(np.asarray([p, len(W)] + list(W), dtype=np.int64).tobytes())
        for b in range(len(W)):
            for arr in (rows[p][b], cols[p][b], mask[p][b]):
                a = np.ascontiguousarray(np.asarray(arr).astype(np.int32))
                h.update(np.asarray(a.shape, dtype=np.int64).tobytes())
                h.update(a.tobytes())
    return h.hexdigest()


def fp32_product_tolerance(want: np.ndarray, row_nnz: np.ndarray) -> np.ndarray:
    """Allowed |got - want| per element of a float32-accumulated product row: abs 1e-4 + rel 1e-5 (the
    benchmark's float32 tolerance) for rows of up to 4096 stored entries; beyond that the absolute
    part grows in proportion to the row length.  A float32 sum of n terms of unit size that is built up
    by chained additions -- a sequential loop, or partial sums committed by atomic adds in whatever
    order they arrive -- rounds each addition to an ulp of a running sum that itself grows like
    sqrt(n), over a number of additions proportional to n: its error grows like n.  A 100 000-entry row
    of U(-1,1) x N(0,1) products has partial sums near 200, one ulp of which is 1.5e-5; 1e-4 absolute is
    seven ulps of the running sum and not attainable by float32 accumulation in any order (SciPy's
    own float32 product misses it too).  How many partial sums a long row is cut into depends on the
    shard size, so the bound is the one that holds for any cut: 2.4e-3 for those rows, against measured
    maxima of 0.4e-3 (one GPU, ~400 partial sums per row) to 1.5e-3 (eight GPUs, ~3000)."""
    n = np.asarray(row_nnz, dtype=np.float64).reshape(-1, 1)
    return 1e-4 * np.maximum(1.0, n / 4096.0) + 1e-5 * np.abs(want)

