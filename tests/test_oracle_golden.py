"""The CPU oracle must reproduce what the unmodified reference produced (tests/golden)."""
import numpy as np
import pytest

from oracle import hyb_oracle as ho
from tests import cases


def _coo(csr):
    rows = np.repeat(np.arange(csr.shape[0], dtype=np.int64), np.diff(csr.indptr))
    return rows, csr.indices.astype(np.int64)


@pytest.mark.parametrize("name", cases.SMALL)
def test_generated_cases(golden, name):
    entry = golden["generated"][name]
    csr = cases.matrix(name)
    assert cases.csr_digest(csr) == entry["csr_digest"], "generator drifted from the golden input"
    row, col = _coo(csr)
    for run in entry["runs"]:
        widths = ho.search_bucket_config(row, col, csr.shape, run["P"], run["N"])
        assert widths == run["widths"]
        r, c, m, v = ho.build_hyb(csr.indptr, csr.indices, csr.shape, widths, csr.data)
        assert ho.digest_hyb(widths, r, c, m) == run["digest"]
        assert [[int(a.shape[0]) for a in rp] for rp in r] == run["ell_rows"]


def test_edge_cases(golden):
    for name, rec in golden["edge"].items():
        csr = cases.edge_csr(rec)
        row, col = _coo(csr)
        if "error" in rec:
            with pytest.raises(ValueError, match="only having 1 non-zero"):
                ho.search_bucket_config(row, col, csr.shape, rec["P"], rec["N"])
            continue
        if rec["forced"]:
            widths = rec["widths"]
        else:
            widths = ho.search_bucket_config(row, col, csr.shape, rec["P"], rec["N"])
            assert widths == rec["widths"], name
        r, c, m, _ = ho.build_hyb(csr.indptr, csr.indices, csr.shape, widths)
        assert ho.digest_hyb(widths, r, c, m) == rec["digest"], name
        r2, c2, m2 = ho.build_hyb_entrywise(csr.indptr, csr.indices, csr.shape, widths)
        assert ho.digest_hyb(widths, r2, c2, m2) == rec["digest"], name
        if "rows" in rec:
            for p in range(len(widths)):
                for b in range(len(widths[p])):
                    assert r[p][b].tolist() == rec["rows"][p][b]
                    assert c[p][b].tolist() == rec["cols"][p][b]
                    assert m[p][b].tolist() == rec["mask"][p][b]


def test_known_edge_shapes(golden):
    e = golden["edge"]
    # a degree-11 row in a width-2 bucket: six ELL rows, same id, last one half padded
    assert e["deg11_width2"]["rows"][0][0][:6] == [0] * 6
    assert e["deg11_width2"]["cols"][0][0][5] == [10, 0] and e["deg11_width2"]["mask"][0][0][5] == [1, 0]
    # an empty partition has no widths; an empty bucket still appears with zero rows
    assert e["empty_partition"]["widths"][1:] == [[], [], []]
    assert e["lone_row_fixup"]["widths"] == [[2, 4, 16]] and e["lone_row_fixup"]["ell_rows"] == [[20, 0, 11]]


def test_row_range_slices_concatenate():
    """A row range yields a contiguous slice of every bucket (what row sharding relies on)."""
    csr = cases.matrix("zipf_2048_s5")
    row, col = _coo(csr)
    for P in (1, 3):
        widths = ho.search_bucket_config(row, col, csr.shape, P, 64)
        whole = ho.build_hyb(csr.indptr, csr.indices, csr.shape, widths, csr.data)
        cuts = [0, 100, 101, 1500, 2048]
        parts = [ho.build_hyb(csr.indptr, csr.indices, csr.shape, widths, csr.data, row_range=(a, b))
                 for a, b in zip(cuts[:-1], cuts[1:])]
        for k in range(4):
            for p in range(P):
                for b in range(len(widths[p])):
                    cat = np.concatenate([part[k][p][b] for part in parts], axis=0)
                    assert np.array_equal(cat, whole[k][p][b])


def test_hyb_product_equals_scipy():
    csr = cases.matrix("skew_8192_s3")
    row, col = _coo(csr)
    B = np.random.default_rng(1).standard_normal((csr.shape[1], 8)).astype(np.float32)
    ref = ho.spmm_scipy(csr.indptr, csr.indices, csr.data, csr.shape, B.astype(np.float64))
    for P in (1, 2):
        widths = ho.search_bucket_config(row, col, csr.shape, P, 32)
        r, c, m, v = ho.build_hyb(csr.indptr, csr.indices, csr.shape, widths, csr.data)
        got = ho.spmm_hyb(r, c, v, csr.shape[0], B)
        np.testing.assert_allclose(got, ref, rtol=1e-6, atol=1e-6)
