"""Host logic of the end-to-end driver mirror (liteform_ae_b200/pipeline.py): feature vectors in the
order the reference's classifiers were trained on (proc05.spmm.end-to-end.py:26-62), the class ->
format mapping (proc05:77), and the routing / fallback decisions of proc05:136-257 with the timed
calls replaced by stand-ins (no GPU here)."""
import math

import numpy as np
import scipy.sparse as sp

from liteform_ae_b200 import pipeline
from liteform_ae_b200.format_matrix_market import MTX


class _Clf:
    def __init__(self, answer):
        self.answer, self.seen = answer, []

    def predict(self, X):
        self.seen.append(np.asarray(X))
        return [self.answer]


def _g():
    rows = np.array([0, 0, 0, 1, 3, 3])
    cols = np.array([0, 2, 4, 1, 0, 3])
    g = MTX(None)
    g.name = "toy"
    g.coo_mtx = sp.coo_matrix((np.ones(6, dtype=np.float32), (rows, cols)), shape=(4, 5))
    return g


def test_feature_vectors_follow_the_reference_order():
    g = _g()
    X = pipeline.get_X_for_format_selection(g, device=None)
    lens = np.array([3, 1, 0, 2])
    np.testing.assert_allclose(X[0], [4, 5, 6, lens.mean(), 0, 3, lens.std()])
    Xp = pipeline.get_X_for_num_partitions(g, 128, device=None)
    np.testing.assert_allclose(Xp[0], [4, 5, 6, lens.mean() / 5, 0, 3 / 5, lens.std() / 5, 128])
    assert len(X) == 1 and X[0].shape == (7,) and Xp[0].shape == (8,)


def test_class_one_means_composed_format():
    g = _g()
    assert pipeline.predict_format_selection(g, _Clf(1), device=None)[0] == "CELL"
    assert pipeline.predict_format_selection(g, _Clf(0), device=None)[0] == "BCSR"
    clf = _Clf(16)
    parts, secs = pipeline.predict_num_partitions(g, clf, 64, device=None)
    assert parts == 16 and secs >= 0 and clf.seen[0].shape == (1, 8) and clf.seen[0][0, -1] == 64


def test_routing_and_fallbacks(monkeypatch):
    g = _g()
    calls = []
    monkeypatch.setattr(pipeline, "_time_composed", lambda g, n, p, d, r: (calls.append(("cell", n, p)), (0.5, 1.25, [[1, 2]]))[1])
    table = pipeline.run([g], _Clf(1), _Clf(4), feat_sizes=(32, 64), device=None)
    assert list(table) == pipeline.TABLE_COLUMNS
    assert table["format"] == ["CELL", "CELL"] and table["num_parts"] == [4, 4]
    assert table["time_exe_our(ms)"] == [1.25, 1.25] and table["time_bucket(s)"] == [0.5, 0.5]
    assert calls == [("cell", 32, 4), ("cell", 64, 4)]

    # a failing composed run is recorded as an infinite time, the sweep goes on
    def boom(*a):
        raise ValueError("The partition is too small, only having 1 non-zero element.")
    monkeypatch.setattr(pipeline, "_time_composed", boom)
    rec = pipeline.run_matrix(g, _Clf(1), _Clf(2), feat_sizes=(32,), device=None)[0]
    assert rec["format"] == "CELL" and math.isinf(rec["time_exe_our(ms)"])

    # class 0: blocks; blocks fail -> CSR; CSR fails too -> CRASHED with time 0
    monkeypatch.setattr(pipeline, "_time_blocks", lambda g, n, bs, d, r: 2.0)
    rec = pipeline.run_matrix(g, _Clf(0), None, feat_sizes=(32,), device=None)[0]
    assert (rec["format"], rec["num_parts"], rec["time_exe_our(ms)"]) == ("BSR", 0, 2.0)
    monkeypatch.setattr(pipeline, "_time_blocks", boom)
    monkeypatch.setattr(pipeline, "_time_csr", lambda g, n, d, r: 3.0)
    rec = pipeline.run_matrix(g, _Clf(0), None, feat_sizes=(32,), device=None)[0]
    assert (rec["format"], rec["time_exe_our(ms)"]) == ("CSR", 3.0)
    monkeypatch.setattr(pipeline, "_time_csr", boom)
    rec = pipeline.run_matrix(g, _Clf(0), None, feat_sizes=(32,), device=None)[0]
    assert (rec["format"], rec["time_exe_our(ms)"]) == ("CRASHED", 0)
