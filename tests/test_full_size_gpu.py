"""Products and block construction at benchmark size (configs 3, 4 and 5), against SciPy in float64.

A full CPU product of these matrices takes minutes, so each case checks (1) the column sums
1^T (A B) == (1^T A) B, which involve every stored entry, and (2) a few thousand sampled rows --
for the skewed matrix all 64 heavy rows -- against the float64 product of exactly those rows.
float32: rel 1e-5 / abs 1e-4; bf16 inputs with fp32 accumulation: rel 1e-2 of the largest
magnitude against the unrounded product, 1e-5 / 1e-4 against the product of the rounded inputs.
Rows with more than 4096 stored entries (the 64 rows of 100 000 entries of the skewed matrix) get
the absolute part scaled by entries / 4096 -- oracle.hyb_oracle.fp32_product_tolerance says
why -- and the test also shows that SciPy's float32 product of those rows is no closer.
"""
import numpy as np
import pytest
import scipy.sparse as sp

from oracle import hyb_oracle as ho
from liteform_ae_b200 import bsr, hyb, synth, width_search as ws
from tests import cases

pytestmark = pytest.mark.gpu

RTOL, ATOL = 1e-5, 1e-4


def _rows_product(csr, pick, B64):
    """float64 product of the rows `pick` of a synth.Csr with B."""
    lens = np.diff(csr.indptr)[pick]
    ptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    idx = np.concatenate([csr.indices[csr.indptr[r]:csr.indptr[r + 1]] for r in pick])
    val = np.concatenate([csr.data[csr.indptr[r]:csr.indptr[r + 1]] for r in pick]).astype(np.float64)
    return np.asarray(sp.csr_matrix((val, idx, ptr), shape=(len(pick), csr.shape[1])) @ B64)


def _check_hyb(csr, N, cuda_device, must_include=()):
    import torch
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    stats, hist = hyb.hyb_stats(d, 1)
    fmt = hyb.build_hyb_device(d, ws.search_from_stats(stats, hist, N, 1), with_mask=False)
    del d
    B = synth.dense_features(csr.shape[1], N, 11)
    Bd = torch.from_numpy(B).to(cuda_device)
    C = torch.full((csr.shape[0], N), float("nan"), device=cuda_device)
    hyb.spmm_hyb(fmt, Bd, out=C)
    assert not torch.isnan(C).any(), "a row of C was not written"
    B64 = B.astype(np.float64)
    colsum_A = np.bincount(csr.indices, weights=csr.data.astype(np.float64), minlength=csr.shape[1])
    got = C.double().sum(dim=0).cpu().numpy()
    # a column of C sums M products; its float32 entries carry ~1e-7 relative error each
    scale = np.abs(csr.data).astype(np.float64).sum() * np.abs(B64).mean()
    assert np.abs(got - colsum_A @ B64).max() <= 1e-6 * scale
    rng = np.random.default_rng(3)
    pick = np.unique(np.concatenate([rng.integers(0, csr.shape[0], 3000), np.asarray(must_include, dtype=np.int64)]))
    got = C[torch.from_numpy(pick).to(cuda_device)].cpu().numpy()
    want = _rows_product(csr, pick, B64)
    lens = np.diff(csr.indptr)[pick]
    err = np.abs(got - want)
    allowed = ho.fp32_product_tolerance(want, lens)
    assert (err <= allowed).all(), f"max excess {(err - allowed).max():.3e} at row length {lens[np.argmax((err - allowed).max(axis=1))]}"
    short = lens <= 4096                       # the benchmark's plain tolerance wherever it is attainable
    np.testing.assert_allclose(got[short], want[short], rtol=RTOL, atol=ATOL)
    if (~short).any():                         # long rows: SciPy accumulating in float32 is no closer to float64
        rows = pick[~short]
        lens_l = np.diff(csr.indptr)[rows]
        ptr = np.concatenate([[0], np.cumsum(lens_l)]).astype(np.int64)
        idx = np.concatenate([csr.indices[csr.indptr[r]:csr.indptr[r + 1]] for r in rows])
        val = np.concatenate([csr.data[csr.indptr[r]:csr.indptr[r + 1]] for r in rows])
        scipy32 = np.asarray(sp.csr_matrix((val, idx, ptr), shape=(len(rows), csr.shape[1])) @ B)
        assert err[~short].max() <= 2.0 * np.abs(scipy32 - want[~short]).max()
    return fmt


def test_config3_uniform_product(cuda_device):
    csr = cases.matrix("uniform32_4194304_s2")
    fmt = _check_hyb(csr, 64, cuda_device)
    assert fmt.bucket_widths == [[32]] and fmt.num_zero_rows == 0


def test_config4_skew_product_all_heavy_rows(cuda_device):
    csr = cases.matrix("skew_1048576_s3")
    lens = np.diff(csr.indptr)
    heavy = np.nonzero(lens >= 100_000)[0]
    assert len(heavy) == 64
    # every heavy row becomes ~100 consecutive ELL rows with one row id, reduced over many thread groups
    _check_hyb(csr, 256, cuda_device, must_include=heavy)


@pytest.fixture(scope="module")
def blocks_full():
    indptr, indices, blocks, shape = synth.banded_blocks()
    return indptr.astype(np.int64), indices, blocks, shape


def _block_rows_product(indptr, indices, blocks64, pick, B_rows64, J):
    """float64 product of the block rows `pick` (rows pick*8 .. pick*8+7) with B, of which only the
    rows of the block columns `J` (sorted; every block column the picked rows touch) are given."""
    cnt = np.diff(indptr)[pick]
    ptr = np.concatenate([[0], np.cumsum(cnt)]).astype(np.int64)
    sel = np.concatenate([np.arange(indptr[I], indptr[I + 1]) for I in pick])
    local = np.searchsorted(J, indices[sel]).astype(np.int32)
    sub = sp.bsr_matrix((blocks64[sel], local, ptr), shape=(len(pick) * 8, len(J) * 8))
    return np.asarray(sub @ B_rows64)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_config5_block_product_real_band(cuda_device, blocks_full, dtype):
    """2^21 rows, band of +-4096 block columns, N in {32, 128, 512}: at N = 512 the four feature tiles
    run one after the other (the order is chosen automatically at this size)."""
    import torch
    indptr, indices, blocks, shape = blocks_full
    tdt = getattr(torch, dtype)
    a = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, dtype, cuda_device)
    rng = np.random.default_rng(5)
    Mb = shape[0] // 8
    pick = np.unique(np.concatenate([rng.integers(0, Mb, 400), [0, 1, Mb - 1]]))
    rows = (pick[:, None] * 8 + np.arange(8)[None, :]).reshape(-1)
    sel = np.concatenate([np.arange(indptr[I], indptr[I + 1]) for I in pick])
    J = np.unique(indices[sel])
    b_rows = torch.from_numpy((J[:, None].astype(np.int64) * 8 + np.arange(8)[None, :]).reshape(-1)).to(cuda_device)
    blocks_r = a.blocks.float().cpu().numpy().astype(np.float64)      # what the kernel multiplies
    # 1^T A as a dense row vector (block column sums scattered to their columns)
    colsum_A = np.zeros(shape[1], dtype=np.float64)
    np.add.at(colsum_A.reshape(-1, 8), indices, blocks_r.sum(axis=1))
    colsum_d = torch.from_numpy(colsum_A).to(cuda_device)
    abs_sum = float(np.abs(blocks_r).sum())
    for N in (32, 128, 512):
        B = synth.dense_features(shape[1], N, 13)
        Bd = torch.from_numpy(B).to(cuda_device).to(tdt)
        C = torch.full((shape[0], N), float("nan"), device=cuda_device)
        bsr.spmm_bsr8(a, Bd, out=C)
        assert not torch.isnan(C).any()
        got = C.double().sum(dim=0)
        want_sum = colsum_d @ Bd.double()                              # float64 on the device: B is large
        scale = abs_sum * float(Bd.float().abs().mean())
        assert float((got - want_sum).abs().max()) <= 1e-6 * scale
        Cs = C[torch.from_numpy(rows).to(cuda_device)].cpu().numpy()
        Br = Bd[b_rows].double().cpu().numpy()
        np.testing.assert_allclose(Cs, _block_rows_product(indptr, indices, blocks_r, pick, Br, J), rtol=RTOL, atol=ATOL)
        if dtype != "float32":      # against the unrounded operands
            want = _block_rows_product(indptr, indices, blocks.astype(np.float64), pick,
                                       B[b_rows.cpu().numpy()].astype(np.float64), J)
            assert np.abs(Cs - want).max() <= 1e-2 * np.abs(want).max()
        del Bd, C, B


def test_config5_device_block_builder_equals_scipy(cuda_device, blocks_full):
    """lf_bsr8_plan / lf_bsr8_fill on the element CSR of the full-size block matrix: the arrays must
    equal what scipy.sparse builds for blocksize (8, 8) -- the reference's block oracle
    (format_matrix_market.py:137) -- bit for bit."""
    import torch
    indptr, indices, blocks, shape = blocks_full
    csr = cases.matrix("blocks_2097152_s4")
    want = csr.toscipy().tobsr(blocksize=(8, 8))
    want.sort_indices()
    assert np.array_equal(want.indptr, indptr) and np.array_equal(want.indices, indices)
    assert np.array_equal(want.data, blocks)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    built = bsr.DeviceBsr8.from_csr_device(d, "float32")
    assert np.array_equal(built.indptr.cpu().numpy(), want.indptr)
    assert np.array_equal(built.indices.cpu().numpy(), want.indices)
    assert torch.equal(built.blocks.cpu(), torch.from_numpy(want.data))
