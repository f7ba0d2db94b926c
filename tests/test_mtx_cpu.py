"""Host-side container: Matrix Market ingestion, features, BSR conversion (no GPU needed)."""
import warnings

import numpy as np
import pytest
import scipy.sparse as sp
from scipy.io import mmwrite

from liteform_ae_b200 import synth
from liteform_ae_b200.format_matrix_market import MTX, Bucket
from oracle import reference_shim as rs


def test_matrix_market_file_forces_unit_values(tmp_path):
    csr = synth.zipf_rows(M=64, seed=3)
    path = tmp_path / "tiny_graph.mtx"
    mmwrite(str(path), csr.toscipy().tocoo())
    g = MTX(str(path))
    assert g.name == "tiny_graph"
    assert g.num_src_nodes() == 64 and g.num_dst_nodes() == 64 and g.num_edges() == csr.nnz
    assert (g.coo_mtx.data == 1).all()          # like the reference, format_matrix_market.py:63-64
    indptr, indices, data = g.adj_tensors("csr")
    assert np.array_equal(indptr, csr.indptr) and np.array_equal(indices, csr.indices)
    with pytest.raises(TypeError):
        g.adj_tensors("ell")
    with pytest.raises(RuntimeError, match="DGL"):
        MTX("cora")


def test_features_and_dot_match_the_reference_container():
    csr = synth.power_law_graph(M=1024, seed=2)
    g = MTX.from_csr(csr.indptr, csr.indices, np.ones(csr.nnz), csr.shape, "pl")
    f = g.matrix_features()
    lens = np.diff(csr.indptr)
    assert f["nnz"] == csr.nnz and f["max_nnz_per_row"] == lens.max() and f["avg_nnz_per_row"] == lens.mean()
    B = np.random.default_rng(0).standard_normal((1024, 4))
    np.testing.assert_allclose(g.dot(B), g.coo_mtx.tocsr() @ B)
    if rs.reference_available():
        warnings.simplefilter("ignore")
        ref = rs.reference_mtx(g.coo_mtx, "pl")
        want = ref.matrix_features()
        assert want.keys() == f.keys()
        for k in want:
            assert want[k] == f[k], k


def test_bsr_with_padding_is_fp16_and_sorted():
    csr = synth.zipf_rows(M=100, seed=1)
    g = MTX.from_csr(csr.indptr, csr.indices, np.ones(csr.nnz), csr.shape)
    b = g.tobsr_with_padding(shape=(128, 128), blocksize=(32, 32))
    assert b.data.dtype == np.float16 and b.blocksize == (32, 32) and b.shape == (128, 128)
    dense = np.zeros((128, 128)); dense[:100, :100] = csr.toscipy().toarray() != 0
    back = sp.bsr_matrix((b.data.astype(np.float32), b.indices, b.indptr), shape=b.shape).toarray()
    assert np.array_equal(back, dense)
    assert str(Bucket(4, 2, 7, [1, 2], {3})).startswith("Bucket(bucket_width=4")


def test_named_graphs_load_from_local_files(tmp_path, monkeypatch):
    """The seven graph names of the reference (format_matrix_market.py:43) resolve to files in
    LITEFORM_DATA_DIR instead of a download; data becomes ones; without a file the error says what to do."""
    import pytest
    import scipy.sparse as sp
    from scipy.io import mmwrite
    from liteform_ae_b200.format_matrix_market import MTX
    a = sp.random(30, 30, density=0.1, format="coo", random_state=3)
    sp.save_npz(tmp_path / "cora.npz", a.tocsr())
    mmwrite(str(tmp_path / "pubmed.mtx"), a)
    monkeypatch.setenv("LITEFORM_DATA_DIR", str(tmp_path))
    for name in ("cora", "pubmed"):
        g = MTX(name)
        assert g.name == name and g.num_edges() == a.nnz and (g.coo_mtx.data == 1).all()
        assert (g.coo_mtx.tocsr() != (a.tocsr() != 0).astype(float)).nnz == 0
    with pytest.raises(RuntimeError, match="LITEFORM_DATA_DIR"):
        MTX("reddit")
