"""Device builder (lf_hyb_stats / lf_hyb_plan / lf_hyb_fill through the C ABI) vs the oracle and
the reference's golden digests: integer work, so every comparison is bit-exact."""
import numpy as np
import pytest

from oracle import hyb_oracle as ho
from liteform_ae_b200 import hyb, width_search as ws
from liteform_ae_b200.format_matrix_market import MTX
from liteform_ae_b200 import format_algos as fa
from tests import cases

pytestmark = pytest.mark.gpu


def _dev(csr, device):
    return hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, device)


def _coo(csr):
    return np.repeat(np.arange(csr.shape[0], dtype=np.int64), np.diff(csr.indptr)), csr.indices.astype(np.int64)


@pytest.mark.parametrize("name", cases.SMALL)
def test_stats_equal_oracle_buckets(cuda_device, name):
    """lf_hyb_stats against counters derived from the oracle's init_buckets (format_algos.py:819-900)."""
    csr = cases.matrix(name)
    d = _dev(csr, cuda_device)
    row, col = _coo(csr)
    for P in (1, 2, 5, 16):
        stats, hist = hyb.hyb_stats(d, P)
        want_s, want_h = ho.bucket_counters(row, col, csr.shape, P)
        assert np.array_equal(stats, want_s)
        assert np.array_equal(hist, want_h)


@pytest.mark.parametrize("name", cases.SMALL)
def test_golden_widths_and_format(cuda_device, golden, name):
    entry = golden["generated"][name]
    csr = cases.matrix(name)
    assert cases.csr_digest(csr) == entry["csr_digest"]
    g = MTX.from_csr(csr.indptr, csr.indices, csr.data, csr.shape, name)
    for run in entry["runs"]:
        widths = fa.search_bucket_config(g, run["P"], fa.CostModelSettings(run["N"], run["P"]), device=cuda_device)
        assert widths == run["widths"]
        rows, cols, mask = fa.build_hyb_format(g, widths, device=cuda_device)
        assert [[int(a.shape[0]) for a in rp] for rp in rows] == run["ell_rows"]
        assert ho.digest_hyb(widths, rows, cols, mask) == run["digest"]


@pytest.mark.parametrize("name", ["zipf_2048_s5", "skew_8192_s3", "powerlaw_8192_s1"])
def test_values_zero_rows_and_padding(cuda_device, name):
    csr = cases.matrix(name)
    row, col = _coo(csr)
    d = _dev(csr, cuda_device)
    for P in (1, 3):
        widths = ho.search_bucket_config(row, col, csr.shape, P, 64)
        fmt = hyb.build_hyb_device(d, widths)
        r, c, m, v = fmt.to_nested_numpy(with_values=True)
        wr, wc, wm, wv = ho.build_hyb(csr.indptr, csr.indices, csr.shape, widths, csr.data)
        count = np.zeros(csr.shape[0], dtype=np.int64)
        for p in range(P):
            for b in range(len(widths[p])):
                assert np.array_equal(r[p][b], wr[p][b])
                assert np.array_equal(c[p][b], wc[p][b])
                assert np.array_equal(m[p][b], wm[p][b])
                assert np.array_equal(v[p][b], wv[p][b])      # values are copied, bit for bit
                count += np.bincount(r[p][b], minlength=csr.shape[0])
        zr = np.sort(fmt.zero_rows.cpu().numpy())
        assert np.array_equal(zr, np.nonzero(count != 1)[0])
        # alignment gaps hold zeros
        cols_flat = fmt.cols.cpu().numpy()
        for i in range(len(fmt.widths)):
            end = fmt.slot_off[i] + fmt.ell_rows[i] * fmt.widths[i]
            assert not cols_flat[end:fmt.slot_off[i + 1]].any()
            assert fmt.slot_off[i] % 64 == 0 and fmt.row_off[i] % 64 == 0


def test_edge_cases(cuda_device, golden):
    for name, rec in golden["edge"].items():
        csr = cases.edge_csr(rec)
        g = MTX.from_csr(csr.indptr, csr.indices, csr.data, csr.shape, name)
        if "error" in rec:
            with pytest.raises(ValueError, match="only having 1 non-zero"):
                fa.search_bucket_config(g, rec["P"], fa.CostModelSettings(rec["N"], rec["P"]), device=cuda_device)
            continue
        if rec["forced"]:
            widths = rec["widths"]
        else:
            widths = fa.search_bucket_config(g, rec["P"], fa.CostModelSettings(rec["N"], rec["P"]), device=cuda_device)
            assert widths == rec["widths"], name
        rows, cols, mask = fa.build_hyb_format(g, widths, device=cuda_device)
        assert ho.digest_hyb(widths, rows, cols, mask) == rec["digest"], name


def test_partition_without_widths_is_rejected(cuda_device):
    csr = cases.matrix("zipf_2048_s5")
    d = _dev(csr, cuda_device)
    with pytest.raises(Exception, match="no bucket width"):
        hyb.build_hyb_device(d, [[1, 2, 4, 8, 16, 32], []])
    with pytest.raises(Exception, match="power of two"):
        hyb.build_hyb_device(d, [[1, 3]])
    with pytest.raises(Exception, match="ascending"):
        hyb.build_hyb_device(d, [[4, 2]])


def test_row_shards_concatenate_to_whole_format(cuda_device):
    csr = cases.matrix("skew_8192_s3")
    row, col = _coo(csr)
    d = _dev(csr, cuda_device)
    for P, G in ((1, 2), (1, 8), (2, 4)):
        widths = ho.search_bucket_config(row, col, csr.shape, P, 128)
        whole = hyb.build_hyb_device(d, widths).to_nested_numpy(with_values=True)
        cuts = hyb.shard_rows(d, G)
        nnz = csr.nnz
        want = [int(np.searchsorted(csr.indptr, (nnz * g) // G, side="left")) for g in range(G)] + [csr.shape[0]]
        assert cuts == want
        parts = [hyb.build_hyb_device(d, widths, row_range=(a, b)).to_nested_numpy(with_values=True)
                 for a, b in zip(cuts[:-1], cuts[1:])]
        for k in range(4):
            for p in range(P):
                for b in range(len(widths[p])):
                    cat = np.concatenate([part[k][p][b] for part in parts], axis=0)
                    assert np.array_equal(cat, whole[k][p][b])


@pytest.mark.parametrize("name", cases.FULL)
def test_full_size_golden_digest(cuda_device, golden, name):
    """Benchmark-size matrices: the device build must hash to what the reference produced."""
    if name not in golden["generated"]:
        pytest.skip("no golden digest recorded for this matrix")
    entry = golden["generated"][name]
    csr = cases.matrix(name)
    assert cases.csr_digest(csr) == entry["csr_digest"]
    d = _dev(csr, cuda_device)
    for run in entry["runs"]:
        stats, hist = hyb.hyb_stats(d, run["P"])
        widths = ws.search_from_stats(stats, hist, run["N"], run["P"])
        assert widths == run["widths"]
        fmt = hyb.build_hyb_device(d, widths)
        rows, cols, mask = fmt.to_nested_numpy()
        assert ho.digest_hyb(widths, rows, cols, mask) == run["digest"]
        del fmt


def test_reusable_workspace_gives_the_same_format(cuda_device):
    """hyb.Workspace: statistics, plan and fill of several matrices out of one growing scratch buffer,
    without the per-call allocation and the final synchronisation -- same counters, same arrays."""
    import torch
    wsp = hyb.Workspace(cuda_device)
    for name, P in (("zipf_2048_s5", 1), ("skew_8192_s3", 3), ("powerlaw_8192_s1", 2), ("zipf_2048_s5", 4)):
        csr = cases.matrix(name)
        d = _dev(csr, cuda_device)
        stats, hist = hyb.hyb_stats(d, P)
        stats_w, hist_w = hyb.hyb_stats(d, P, workspace=wsp)
        assert np.array_equal(stats, stats_w) and np.array_equal(hist, hist_w)
        widths = ws.search_from_stats(stats, hist, 64, P)
        a = hyb.build_hyb_device(d, widths)
        b = hyb.build_hyb_device(d, widths, workspace=wsp)
        torch.cuda.synchronize(cuda_device)
        for x, y in ((a.rows, b.rows), (a.cols, b.cols), (a.vals, b.vals), (a.mask, b.mask), (a.zero_rows, b.zero_rows)):
            assert torch.equal(x, y)
        assert np.array_equal(a.ell_rows, b.ell_rows) and np.array_equal(a.slot_off, b.slot_off)
