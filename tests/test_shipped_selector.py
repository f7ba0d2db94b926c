"""The format-selection model the reference ships (playground_pipline/models/
model.for_selection.train_set.RandomForest.joblib, loaded at proc05.spmm.end-to-end.py:115, used at
proc05:65-79) run through this package's pipeline.  Needs the reference checkout (environment
variable LITEFORM_REFERENCE_ROOT) and joblib; skipped otherwise.  What is checked: the pipeline feeds
the model the seven columns it was fitted on, in the order of proc05:26-47, with the values the
reference's own MTX.matrix_features (format_matrix_market.py:153-202) computes, so both drivers
get the same answer from the same model."""
import os
import warnings

import numpy as np
import pytest

from oracle import reference_shim as rs
from liteform_ae_b200 import pipeline
from liteform_ae_b200.format_matrix_market import MTX
from tests import cases

joblib = pytest.importorskip("joblib")
MODEL = os.path.join(os.environ.get("LITEFORM_REFERENCE_ROOT", ""), "playground_pipline", "models",
                     "model.for_selection.train_set.RandomForest.joblib")
needs_model = pytest.mark.skipif(not (rs.reference_available() and os.path.isfile(MODEL)),
                                 reason="no reference checkout with the shipped model on this machine")

# proc05.spmm.end-to-end.py:28-36, in that order
REFERENCE_COLUMNS = ["num_rows", "num_cols", "nnz", "avg_nnz_per_row", "min_nnz_per_row", "max_nnz_per_row",
                     "std_dev_nnz_per_row"]


def _load():
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")          # pickled by an older scikit-learn
        return joblib.load(MODEL)


def _mtx(name):
    csr = cases.matrix(name)
    return MTX.from_csr(csr.indptr, csr.indices, csr.data, csr.shape, name), csr


@needs_model
@pytest.mark.parametrize("name", ["zipf_16384_s0", "blocks_4096_s4", "powerlaw_8192_s1"])
def test_shipped_model_gets_the_reference_feature_vector(name):
    clf = _load()
    assert getattr(clf, "n_features_in_", 7) == 7
    assert pipeline.FORMAT_SELECTION_FEATURES == REFERENCE_COLUMNS
    g, csr = _mtx(name)
    ref_g = rs.reference_mtx(csr.tocoo(), name)
    ref_feat = ref_g.matrix_features()
    want_X = [np.array([ref_feat[c] for c in REFERENCE_COLUMNS])]
    X = pipeline.get_X_for_format_selection(g, device=None)
    np.testing.assert_allclose(X[0], want_X[0], rtol=1e-12)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        fmt, seconds = pipeline.predict_format_selection(g, clf, device=None)
        want = "CELL" if clf.predict(want_X)[0] == 1 else "BCSR"       # proc05:77
    assert fmt == want and fmt in ("CELL", "BCSR") and seconds >= 0


@needs_model
@pytest.mark.gpu
@pytest.mark.parametrize("name", ["zipf_16384_s0", "blocks_4096_s4"])
def test_shipped_model_routes_the_same_on_device_features(cuda_device, name):
    """Row statistics from lf_row_stats instead of the reference's Python loop: same vector, same class."""
    clf = _load()
    g, _ = _mtx(name)
    X_host = pipeline.get_X_for_format_selection(g, device=None)
    X_dev = pipeline.get_X_for_format_selection(g, device=cuda_device)
    np.testing.assert_allclose(X_dev[0], X_host[0], rtol=1e-12)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        assert pipeline.predict_format_selection(g, clf, device=cuda_device)[0] == \
            pipeline.predict_format_selection(g, clf, device=None)[0]
