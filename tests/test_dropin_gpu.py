"""The reference pipeline's call sequence (proc05.spmm.end-to-end.py:154-176) on the drop-in modules."""
import numpy as np
import pytest

from liteform_ae_b200 import synth
from liteform_ae_b200.format_algos import (CostModelSettings, bench_hyb_with_config, bench_naive,
                                           build_hyb_format, search_bucket_config, spmm)
from liteform_ae_b200.format_matrix_market import MTX
from oracle import hyb_oracle as ho

pytestmark = pytest.mark.gpu


def _graph(M=4096, seed=7):
    csr = synth.power_law_graph(M=M, seed=seed)
    import scipy.sparse as sp
    g = MTX(None)                        # the reference's hook for in-memory matrices
    g.name = "synthetic"
    g.coo_mtx = sp.coo_matrix((np.ones(csr.nnz), (np.repeat(np.arange(M), np.diff(csr.indptr)), csr.indices)),
                              shape=csr.shape)
    return g, csr


@pytest.mark.parametrize("num_parts", [1, 4])
def test_pipeline_sequence(cuda_device, num_parts):
    import torch
    g, csr = _graph()
    for num_features in (32, 128):
        cfg = CostModelSettings(feat_size=num_features, num_parts=num_parts)
        assert str(cfg) == f"(feat_size={num_features}, num_parts={num_parts})"
        bucket_config = search_bucket_config(g, num_parts, cfg)
        coo = g.coo_mtx
        assert bucket_config == ho.search_bucket_config(coo.row, coo.col, coo.shape, num_parts, num_features)
        x = torch.ones((g.num_dst_nodes(), num_features))
        y_ndarray = g.dot(x.numpy())
        hyb_format = build_hyb_format(g, bucket_config)
        want = ho.build_hyb(csr.indptr, csr.indices, csr.shape, bucket_config)
        assert ho.digest_hyb(bucket_config, *hyb_format) == ho.digest_hyb(bucket_config, *want[:3])
        ms = bench_hyb_with_config(g, x, y_ndarray, feat_size=num_features, bucket_widths=bucket_config,
                                   bucketing_format=hyb_format, coarsening_factor=2, num_col_parts=num_parts,
                                   use_implicit_unroll=True, check_correctness=True, warmup=1, repeat=3)
        assert ms > 0
        C = spmm(g, x, bucket_widths=bucket_config)
        np.testing.assert_allclose(C.cpu().numpy(), y_ndarray, rtol=1e-5, atol=1e-4)


def test_bench_naive_and_wrong_answer_detection(cuda_device):
    import torch
    g, _ = _graph(M=2048, seed=8)
    x = torch.rand((g.num_dst_nodes(), 64))
    y = g.dot(x.numpy())
    assert bench_naive(g, x, y, feat_size=64, coarsening_factor=2, check_correctness=True, warmup=1, repeat=2) > 0
    with pytest.raises(AssertionError):
        bench_naive(g, x, y + 1.0, feat_size=64, check_correctness=True, warmup=0, repeat=1)


def test_duplicate_entries_are_refused(cuda_device):
    import scipy.sparse as sp
    g = MTX(None)
    g.coo_mtx = sp.coo_matrix((np.ones(3), ([0, 0, 1], [1, 1, 0])), shape=(2, 2))
    with pytest.raises(ValueError, match="duplicate"):
        search_bucket_config(g, 1, CostModelSettings(32, 1))


def test_matrix_features_device_matches_host(cuda_device):
    g, _ = _graph(M=8192, seed=9)
    host, dev = g.matrix_features(), g.matrix_features_device(cuda_device)
    assert host.keys() == dev.keys()
    for k, v in host.items():
        if k == "name":
            assert dev[k] == v
        elif k.startswith("std_dev"):
            assert dev[k] == pytest.approx(float(v), rel=1e-12)
        else:
            assert float(dev[k]) == float(v), k
