"""Host width search on counter-form statistics (derived from the oracle's ``init_buckets``, which
is pinned to format_algos.py:819-900) vs the oracle's set-based search."""
import numpy as np
import pytest

from oracle import hyb_oracle as ho
from liteform_ae_b200 import synth, width_search as ws
from tests import cases


def _coo(csr):
    return np.repeat(np.arange(csr.shape[0], dtype=np.int64), np.diff(csr.indptr)), csr.indices.astype(np.int64)


@pytest.mark.parametrize("name", ["zipf_2048_s5", "powerlaw_8192_s1", "skew_8192_s3", "uniform32_4096_s2"])
def test_search_from_stats_equals_oracle(name):
    csr = cases.matrix(name)
    row, col = _coo(csr)
    for P in (1, 2, 7):
        stats, hist = ho.bucket_counters(row, col, csr.shape, P)
        for N in (32, 512):
            assert ws.search_from_stats(stats, hist, N, P) == ho.search_bucket_config(row, col, csr.shape, P, N)


def test_stats_tables_equal_oracle_buckets():
    csr = synth.skewed_rows(M=4096, seed=8, heavy_rows=4, heavy_len=3000)
    row, col = _coo(csr)
    for P in (1, 3):
        stats, hist = ho.bucket_counters(row, col, csr.shape, P)
        pools = ho.init_buckets(row, col, csr.shape, P)
        bins = np.arange(ws.BINS)
        for p, pool in enumerate(pools):
            for k in range(ws.NUM_CLASSES):
                b = pool.get(1 << k)
                if b is None:
                    assert stats[p, k].tolist() == [0, 0, 0]
                    continue
                assert stats[p, k].tolist() == [b.num_rows, b.nnz, len(b.row_ids)]
                assert int(hist[p][(bins >> k) & 1 == 1].sum()) == len(b.cols)


def test_edge_cases_from_golden(golden):
    for name, rec in golden["edge"].items():
        if rec.get("forced"):
            continue
        csr = cases.edge_csr(rec)
        row, col = _coo(csr)
        stats, hist = ho.bucket_counters(row, col, csr.shape, rec["P"])
        if "error" in rec:
            with pytest.raises(ValueError, match="only having 1 non-zero"):
                ws.search_from_stats(stats, hist, rec["N"], rec["P"])
        else:
            assert ws.search_from_stats(stats, hist, rec["N"], rec["P"]) == rec["widths"], name
