"""Drop-in surface of the reference's ``format_algos`` module, backed by the sm_100a library.

Same names, argument meaning and error behaviour as playground_pipline/format_algos.py
(``__all__`` at format_algos.py:26-31) so that the calling sequence of the reference pipeline
(proc05.spmm.end-to-end.py:154-176) runs unchanged:

    cfg  = CostModelSettings(feat_size=K, num_parts=P)
    bc   = search_bucket_config(g, P, cfg)
    hyb  = build_hyb_format(g, bc)
    ms   = bench_hyb_with_config(g, x, y, feat_size=K, bucket_widths=bc, bucketing_format=hyb,
                                 coarsening_factor=2, num_col_parts=P, use_implicit_unroll=True)

Additions (the reference never returns the product): ``build_hyb_format_device`` keeps the
format in device memory, ``spmm`` returns C.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np

from . import hyb as _hyb
from . import width_search as _ws
from .format_matrix_market import MTX
from .timing import profile_ms

__all__ = ["build_hyb_format", "bench_hyb_with_config", "search_bucket_config", "CostModelSettings",
           "bench_bsrmm", "bench_naive", "build_hyb_format_device", "spmm", "suggest_num_parts"]


class CostModelSettings:
    def __init__(self, feat_size: int, num_parts: int):
        self.feat_size = feat_size
        self.num_parts = num_parts

    def __str__(self) -> str:
        return F"(feat_size={self.feat_size}, num_parts={self.num_parts})"


def search_bucket_config(g: MTX, num_parts: int, cost_model_config: CostModelSettings,
                         device="cuda") -> List[List[int]]:
    """Bucket widths per column partition (format_algos.py:988-1032).

    The per-nonzero statistics run on the device (``lf_hyb_stats``); the O(#classes^2) search
    runs on the host on those counters.  Raises ``ValueError`` for a partition that holds a
    single nonzero, like the reference (format_algos.py:920-921).
    """
    csr = g.csr_device(device)
    stats, hist = _hyb.hyb_stats(csr, int(num_parts))
    return _ws.search_from_stats(stats, hist, int(cost_model_config.feat_size),
                                 int(cost_model_config.num_parts))


def suggest_num_parts(g: MTX, feat_size: int, candidates=(1, 2, 4, 8, 16, 32), device="cuda"):
    """Number of column partitions with the smallest modelled memory traffic.

    NOT a reference-pinned function: the reference takes ``num_parts`` from a RandomForest whose model
    file is not part of its repository (proc05.spmm.end-to-end.py:82-97, 142-148).  This chooser
    evaluates the reference's own cost model (format_algos.py:1035-1166) at its best widths for every
    candidate and sums it over the partitions; candidates that leave a partition with a single
    nonzero are skipped.  Returns ``(num_parts, {candidate: cost})``."""
    csr = g.csr_device(device)
    costs = {}
    for P in candidates:
        if P > g.num_dst_nodes():
            continue
        stats, hist = _hyb.hyb_stats(csr, int(P))
        per_part = []
        try:
            _ws.search_from_stats(stats, hist, int(feat_size), int(P), cost_out=per_part)
        except ValueError:
            continue
        costs[int(P)] = float(sum(per_part))
    if not costs:
        raise ValueError("no candidate number of partitions is usable")
    return min(costs, key=costs.get), costs


def build_hyb_format_device(g: MTX, bucket_widths: Sequence[Sequence[int]], row_range=None,
                            device="cuda", with_mask: bool = True) -> _hyb.HybFormat:
    """The format of ``build_hyb_format`` left in device memory (plus a values array)."""
    return _hyb.build_hyb_device(g.csr_device(device), bucket_widths, row_range, with_mask)


def build_hyb_format(g: MTX, bucket_widths: Sequence[Sequence[int]], device="cuda"):
    """``(row_indices_nd, col_indices_nd, mask_nd)``, nested ``[partition][bucket]`` NumPy arrays
    of shapes ``(R,)``, ``(R, w)``, ``(R, w)`` (format_algos.py:226-237, 385), built on the device."""
    return build_hyb_format_device(g, bucket_widths, device=device).to_nested_numpy()


def _as_format(g: MTX, bucket_widths, bucketing_format, device) -> _hyb.HybFormat:
    if isinstance(bucketing_format, _hyb.HybFormat):
        return bucketing_format
    rows_nd, cols_nd = bucketing_format[0], bucketing_format[1]
    # a 4th element carries values; otherwise the 0/1 mask is the value array, which is what the
    # reference uploads as A (format_algos.py:568-570)
    vals_nd = bucketing_format[3] if len(bucketing_format) > 3 else bucketing_format[2]
    shape = (g.num_src_nodes(), g.num_dst_nodes())
    return _hyb.HybFormat.from_nested_numpy(bucket_widths, rows_nd, cols_nd, vals_nd, shape, device)


def _dense_to_device(x, device):
    import torch
    t = x if isinstance(x, torch.Tensor) else torch.as_tensor(np.asarray(x))
    return t.to(device=device, dtype=torch.float32).contiguous()


def spmm(a, B, out=None, accumulate: bool = False, bucket_widths=None, device="cuda"):
    """C = A @ B on the device.  ``a`` is a ``HybFormat`` or an ``MTX`` (then ``bucket_widths``
    selects the format; default: searched with P=1)."""
    if isinstance(a, MTX):
        if bucket_widths is None:
            n = int(B.shape[1])
            bucket_widths = search_bucket_config(a, 1, CostModelSettings(n, 1), device)
        a = build_hyb_format_device(a, bucket_widths, device=device, with_mask=False)
    return _hyb.spmm_hyb(a, _dense_to_device(B, a.device), out=out, accumulate=accumulate)


def bench_hyb_with_config(g, x, y_ndarray, feat_size=128, bucket_widths=[], bucketing_format=[],
                          coarsening_factor=2, num_col_parts=1, use_implicit_unroll=False,
                          check_correctness=False, device="cuda", warmup=10, repeat=100) -> float:
    """Upload the format and B, run the SpMM, return its mean time in milliseconds
    (format_algos.py:388-605).  ``coarsening_factor`` and ``use_implicit_unroll`` steer the
    reference's code generator and have no effect here; ``check_correctness`` compares with
    ``y_ndarray`` at rtol 1e-4 like format_algos.py:596-597."""
    import torch
    assert len(bucket_widths) == num_col_parts, "one width list per column partition"
    fmt = _as_format(g, bucket_widths, bucketing_format, device)
    B = _dense_to_device(x, fmt.device).reshape(-1, feat_size)
    C = torch.empty((fmt.row_end - fmt.row_begin, feat_size), dtype=torch.float32, device=fmt.device)
    _hyb.spmm_hyb(fmt, B, out=C)
    if check_correctness:
        np.testing.assert_allclose(C.cpu().numpy(), np.asarray(y_ndarray).reshape(-1, feat_size),
                                   rtol=1e-4, atol=1e-4)
    dur = profile_ms(lambda: _hyb.spmm_hyb(fmt, B, out=C), warmup=warmup, repeat=repeat)
    print("cell exe time: {:.6f} ms".format(dur))
    return dur


def bench_naive(g, x, y_ndarray, feat_size=128, coarsening_factor=2, check_correctness=False,
                device="cuda", warmup=10, repeat=100) -> float:
    """CSR SpMM timing (format_algos.py:1689-1755).  The reference feeds the CSC arrays of A to
    a CSR kernel (format_algos.py:1698), which is A^T B for a non-symmetric A; this computes A B."""
    import torch
    csr = g.csr_device(device)
    B = _dense_to_device(x, csr.indptr.device).reshape(-1, feat_size)
    C = torch.empty((csr.shape[0], feat_size), dtype=torch.float32, device=B.device)
    _hyb.spmm_csr(csr, B, out=C)
    if check_correctness:
        np.testing.assert_allclose(C.cpu().numpy(), np.asarray(y_ndarray).reshape(-1, feat_size),
                                   rtol=1e-4, atol=1e-4)
    dur = profile_ms(lambda: _hyb.spmm_csr(csr, B, out=C), warmup=warmup, repeat=repeat)
    print("naive exe time: {:.6f} ms".format(dur))
    return dur


def bench_bsrmm(bsr_mat, x, block_size, device="cuda", warmup=10, repeat=100) -> float:
    """Block-sparse SpMM timing (format_algos.py:1562-1643)."""
    from . import bsr as _bsr
    return _bsr.bench_bsrmm(bsr_mat, x, block_size, device=device, warmup=warmup, repeat=repeat)
