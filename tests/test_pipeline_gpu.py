"""The end-to-end driver mirror on a GPU: both branches run on the device paths and give finite
times; the block branch computes what SciPy computes on the padded matrix."""
import numpy as np
import pytest
import scipy.sparse as sp

from liteform_ae_b200 import bsr, format_algos as fa, pipeline, synth
from liteform_ae_b200.format_matrix_market import MTX

pytestmark = pytest.mark.gpu


class _Clf:
    def __init__(self, answer):
        self.answer = answer

    def predict(self, X):
        assert np.asarray(X).ndim == 2
        return [self.answer]


def _g():
    csr = synth.zipf_rows(M=2048, seed=5)
    return MTX.from_csr(csr.indptr, csr.indices, csr.data, csr.shape, "zipf_2048"), csr


def test_composed_branch(cuda_device):
    g, _ = _g()
    table = pipeline.run([g], _Clf(1), _Clf(2), feat_sizes=(32, 64), device=cuda_device, repeat=3)
    assert table["format"] == ["CELL", "CELL"] and table["num_parts"] == [2, 2]
    assert all(np.isfinite(t) and t > 0 for t in table["time_exe_our(ms)"])
    # without the reference's partition model the package's own chooser answers
    rec = pipeline.run_matrix(g, _Clf(1), None, feat_sizes=(32,), device=cuda_device, repeat=3)[0]
    assert rec["num_parts"] >= 1 and np.isfinite(rec["time_exe_our(ms)"])


def test_block_and_csr_branches(cuda_device, monkeypatch):
    import torch
    g, csr = _g()
    table = pipeline.run([g], _Clf(0), None, feat_sizes=(32, 128), device=cuda_device, repeat=3)
    assert table["format"] == ["BSR", "BSR"] and table["num_parts"] == [0, 0]
    assert all(np.isfinite(t) and t > 0 for t in table["time_exe_our(ms)"])
    # what the block branch computes: the product on the matrix padded to a square multiple of 32
    a = g.tobsr_device(shape=(2048, 2048), dtype="float16", device=cuda_device)
    x = torch.rand(2048, 32).half().to(cuda_device)
    got = bsr.spmm_bsr8(a, x).cpu().numpy()
    A16 = sp.csr_matrix((csr.data.astype(np.float16).astype(np.float64), csr.indices, csr.indptr), shape=csr.shape)
    np.testing.assert_allclose(got, A16 @ x.float().cpu().numpy().astype(np.float64), rtol=1e-4, atol=1e-3)
    # block conversion fails -> CSR product
    def boom(*a, **k):
        raise MemoryError("no room for the blocks")
    monkeypatch.setattr(MTX, "tobsr_device", boom)
    rec = pipeline.run_matrix(g, _Clf(0), None, feat_sizes=(64,), device=cuda_device, repeat=3)[0]
    assert rec["format"] == "CSR" and np.isfinite(rec["time_exe_our(ms)"]) and rec["time_exe_our(ms)"] > 0


@pytest.mark.parametrize("name,N", [("powerlaw", 128), ("uniform", 64), ("skew", 256)])
def test_partition_chooser_is_close_to_the_measured_best(cuda_device, name, N):
    """format_algos.suggest_num_parts is this package's stand-in for the partition-count model the
    reference's checkout lacks (proc05.spmm.end-to-end.py:82-97); it is not reference-pinned, so it
    is validated by measurement: on mid-size variants of the benchmark matrices the product at the
    chosen partition count must take at most 15 % longer than the fastest of P in {1, 2, 4, 8, 16}.
    (At full benchmark size the chosen P = 1 is the measured best on all four matrices; on the
    quarter-size skewed matrix, whose B slices fit the L2 at P = 4, P = 4 measured 12 % faster than
    the chosen P = 1 -- the cost model knows no cache capacity.)"""
    import statistics
    import torch
    from liteform_ae_b200 import hyb, synth, width_search as ws
    from liteform_ae_b200.timing import time_ms
    make = {"powerlaw": lambda: synth.power_law_graph(M=1 << 18, seed=1),
            "uniform": lambda: synth.uniform_rows(M=1 << 19, seed=2),
            "skew": lambda: synth.skewed_rows(M=1 << 18, seed=3, heavy_rows=16, heavy_len=30000)}[name]
    csr = make()
    g = MTX.from_csr(csr.indptr, csr.indices, csr.data, csr.shape, name)
    pick, costs = fa.suggest_num_parts(g, N, candidates=(1, 2, 4, 8, 16), device=cuda_device)
    d = g.csr_device(cuda_device)
    B = torch.randn((csr.shape[1], N), device=cuda_device)
    C = torch.empty((csr.shape[0], N), device=cuda_device)
    ms = {}
    for P in costs:
        stats, hist = hyb.hyb_stats(d, P)
        fmt = hyb.build_hyb_device(d, ws.search_from_stats(stats, hist, N, P), with_mask=False)
        ms[P] = statistics.median(time_ms(lambda: hyb.spmm_hyb(fmt, B, out=C), warmup=5, repeat=30, flush_l2=True))
        del fmt
    best = min(ms.values())
    assert ms[pick] <= 1.15 * best, f"chooser picked P={pick} ({ms[pick]:.3f} ms), measured {ms}"
