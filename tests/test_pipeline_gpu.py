"""The end-to-end driver mirror on a GPU: both branches run on the device paths and give finite
times; the block branch computes what SciPy computes on the padded matrix."""
import numpy as np
import pytest
import scipy.sparse as sp

from liteform_ae_b200 import bsr, pipeline, synth
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
