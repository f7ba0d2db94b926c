"""Run the unmodified reference next to the oracle (only where a reference checkout exists)."""
import warnings

import pytest

from oracle import hyb_oracle as ho
from oracle import reference_shim as rs
from liteform_ae_b200 import synth

pytestmark = pytest.mark.skipif(not rs.reference_available(), reason="no reference checkout on this machine")


@pytest.mark.parametrize("gen,M,seed", [
    ("zipf_rows", 512, 11), ("zipf_rows", 3000, 12), ("power_law_graph", 2048, 13),
    ("skewed_rows", 2048, 14), ("uniform_rows", 1024, 15)])
def test_oracle_matches_reference(gen, M, seed):
    warnings.simplefilter("ignore")
    fa, _ = rs.load_reference()
    csr = getattr(synth, gen)(M=M, seed=seed)
    coo = csr.tocoo()
    g = rs.reference_mtx(coo)
    for P in (1, 2, 5):
        for N in (32, 256):
            try:
                want = fa.search_bucket_config(g, P, fa.CostModelSettings(N, P))
            except ValueError as e:
                with pytest.raises(ValueError, match=str(e)[:20]):
                    ho.search_bucket_config(coo.row, coo.col, coo.shape, P, N)
                continue
            got = ho.search_bucket_config(coo.row, coo.col, coo.shape, P, N)
            assert got == want
            r, c, m = fa.build_hyb_format(g, want)
            r2, c2, m2, _ = ho.build_hyb(csr.indptr, csr.indices, csr.shape, want, csr.data)
            assert ho.digest_hyb(want, r, c, m) == ho.digest_hyb(want, r2, c2, m2)


def test_cost_scalar_matches_reference():
    """The float the search compares must be bit-identical, not just the winning widths."""
    warnings.simplefilter("ignore")
    fa, _ = rs.load_reference()
    csr = synth.zipf_rows(M=4096, seed=21)
    coo = csr.tocoo()
    g = rs.reference_mtx(coo)
    for P in (1, 4):
        ref_pools = fa.get_init_buckets(g, P)
        my_pools = ho.init_buckets(coo.row, coo.col, coo.shape, P)
        cfg = fa.CostModelSettings(96, P)
        for rp, mp in zip(ref_pools, my_pools):
            assert list(rp.keys()) == list(mp.keys())
            assert fa.get_memory_cost(rp, cfg)["cost"] == ho.memory_cost(mp, 96, P)
