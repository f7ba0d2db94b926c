"""Statistics pass on matrices made of very long rows.  Row segments of 2048 entries or more are
listed and marked by a second, grid-wide kernel; the list holds 8192 segments and further ones are
marked in place.  8300 rows of 8192 consecutive columns exercise the deferred path, the overflow
path and (with two partitions) their mixture with ordinary segments.  Expected counters follow from
the segment lengths alone (format_algos.py:875-896: width 2^ceil(log2 deg), capped at 1024 with
deg-dependent row estimate), expected class masks from interval coverage."""
import numpy as np
import pytest

from liteform_ae_b200 import hyb

pytestmark = pytest.mark.gpu

K, LEN, ROWS = 16384, 8192, 8300


def _expected(starts, P):
    psz = -(-K // P)
    stats = np.zeros((P, 11, 3), dtype=np.int64)
    cover = np.zeros((11, K + 1), dtype=np.int64)          # per class: difference array over columns
    for p in range(P):
        lo = np.maximum(starts, p * psz)
        hi = np.minimum(starts + LEN, min((p + 1) * psz, K))
        deg = np.maximum(hi - lo, 0)
        live = deg > 0
        k = np.zeros_like(deg)
        k[live] = np.ceil(np.log2(deg[live])).astype(np.int64)
        kc = np.minimum(k, 10)
        reps = np.where(k > 10, 1 << np.maximum(k - 10, 0), 1)
        for c in range(11):
            sel = live & (kc == c)
            stats[p, c] = (reps[sel].sum(), deg[sel].sum(), sel.sum())
            np.add.at(cover[c], lo[sel], 1)
            np.add.at(cover[c], hi[sel], -1)
    mask = np.zeros(K, dtype=np.int64)
    for c in range(11):
        mask |= (np.cumsum(cover[c])[:K] > 0).astype(np.int64) << c
    hist = np.zeros((P, 2048), dtype=np.int64)
    cols = np.arange(K)
    np.add.at(hist, (cols[mask > 0] // psz, mask[mask > 0]), 1)
    return stats, hist


@pytest.mark.parametrize("P", [1, 2, 3])
def test_more_long_segments_than_the_list_holds(cuda_device, P):
    import torch
    starts = (np.arange(ROWS, dtype=np.int64) * 37) % (K - LEN + 1)
    d_starts = torch.from_numpy(starts).to(cuda_device)
    indices = (d_starts[:, None] + torch.arange(LEN, device=cuda_device)[None, :]).to(torch.int32).reshape(-1).contiguous()
    indptr = torch.arange(ROWS + 1, dtype=torch.int64, device=cuda_device) * LEN
    csr = hyb.DeviceCsr(indptr, indices, None, (ROWS, K))
    want_stats, want_hist = _expected(starts, P)
    for _ in range(2):                                     # the second call reuses nothing of the first
        stats, hist = hyb.hyb_stats(csr, P)
        np.testing.assert_array_equal(stats, want_stats)
        np.testing.assert_array_equal(hist, want_hist)
