"""Randomised small cases (seeded): non-square shapes, arbitrary partition counts and feature
widths, row ranges, forced width lists.  Format bit-exact against the oracle, products against
SciPy in float64."""
import numpy as np
import pytest
import scipy.sparse as sp

from oracle import hyb_oracle as ho
from liteform_ae_b200 import hyb, synth, width_search as ws

pytestmark = pytest.mark.gpu


def _random_csr(rng, M, K, density):
    A = sp.random(M, K, density=density, format="csr", random_state=np.random.RandomState(int(rng.integers(1 << 30))),
                  data_rvs=lambda n: rng.uniform(-1, 1, n))
    A.sort_indices()
    return synth.Csr(A.indptr.astype(np.int64), A.indices.astype(np.int32), A.data.astype(np.float32), (M, K))


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes(cuda_device, seed):
    import torch
    rng = np.random.default_rng(1000 + seed)
    for _ in range(6):
        M, K = int(rng.integers(1, 400)), int(rng.integers(1, 400))
        csr = _random_csr(rng, M, K, float(rng.choice([0.002, 0.02, 0.2, 0.9])))
        P = int(rng.integers(1, min(K, 9) + 1))
        N = int(rng.choice([1, 4, 7, 32, 36, 64, 128, 260]))
        rows = np.repeat(np.arange(M, dtype=np.int64), np.diff(csr.indptr))
        d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
        st, hi = hyb.hyb_stats(d, P)
        want_st, want_hi = ho.bucket_counters(rows, csr.indices.astype(np.int64), csr.shape, P)
        assert np.array_equal(st, want_st) and np.array_equal(hi, want_hi)
        try:
            widths = ho.search_bucket_config(rows, csr.indices.astype(np.int64), csr.shape, P, max(N, 1))
        except ValueError:
            with pytest.raises(ValueError):
                ws.search_from_stats(st, hi, max(N, 1), P)
            # forced widths instead: one random ascending list per non-empty partition
            psz = -(-K // P)
            widths = [sorted(set(int(1 << k) for k in rng.integers(0, 7, 3))) if ((csr.indices // psz) == p).any() else []
                      for p in range(P)]
        else:
            assert ws.search_from_stats(st, hi, max(N, 1), P) == widths
        a, b = sorted(int(x) for x in rng.integers(0, M + 1, 2))
        for rr in ((0, M), (a, b)):
            fmt = hyb.build_hyb_device(d, widths, row_range=rr)
            r, c, m, v = fmt.to_nested_numpy(with_values=True)
            wr, wc, wm, wv = ho.build_hyb(csr.indptr, csr.indices, csr.shape, widths, csr.data, row_range=rr)
            assert ho.digest_hyb(widths, r, c, m) == ho.digest_hyb(widths, wr, wc, wm)
            for p in range(P):
                for k in range(len(widths[p])):
                    assert np.array_equal(v[p][k], wv[p][k])
            B = rng.standard_normal((K, N)).astype(np.float32)
            Bd = torch.from_numpy(B).to(cuda_device)
            want = (csr.toscipy().astype(np.float64) @ B.astype(np.float64))[rr[0]:rr[1]]
            C = torch.full((rr[1] - rr[0], N), float("nan"), device=cuda_device)
            hyb.spmm_hyb(fmt, Bd, out=C)
            np.testing.assert_allclose(C.cpu().numpy(), want, rtol=1e-5, atol=1e-4)
            C2 = torch.full((rr[1] - rr[0], N), float("nan"), device=cuda_device)
            hyb.spmm_csr(d, Bd, out=C2, row_range=rr)
            np.testing.assert_allclose(C2.cpu().numpy(), want, rtol=1e-5, atol=1e-4)
