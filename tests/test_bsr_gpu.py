"""8x8 block SpMM through the C ABI vs SciPy's BSR product (the reference's block format oracle).

float32: rel 1e-5 / abs 1e-4 against the float64 product.  16-bit inputs with fp32 accumulate:
rel 1e-2 against the float64 product of the unrounded inputs, and (tighter, isolating the
accumulation) 1e-5 against the float64 product of the rounded inputs."""
import numpy as np
import pytest
import scipy.sparse as sp

from liteform_ae_b200 import bsr, synth

pytestmark = pytest.mark.gpu


def _case(M, seed, per_row=8):
    indptr, indices, blocks, shape = synth.banded_blocks(M=M, seed=seed, per_block_row=per_row, half_band=64)
    A = sp.bsr_matrix((blocks.astype(np.float64), indices, indptr), shape=shape)
    return indptr, indices, blocks, shape, A


@pytest.mark.parametrize("N", [4, 20, 32, 36, 64, 100, 128, 256, 512])
def test_bsr8_f32_matches_scipy(cuda_device, N):
    import torch
    indptr, indices, blocks, shape, A = _case(2048, 4)
    B = synth.dense_features(shape[1], N, 0)
    a = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, "float32", cuda_device)
    C = bsr.spmm_bsr8(a, torch.from_numpy(B).to(cuda_device)).cpu().numpy()
    np.testing.assert_allclose(C, A @ B.astype(np.float64), rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
@pytest.mark.parametrize("N", [8, 24, 32, 40, 64, 72, 128, 256, 512])
def test_bsr8_16bit_matches_scipy(cuda_device, dtype, N):
    import torch
    tdt = getattr(torch, dtype)
    for per_row in (8, 5):          # 5: odd block count exercises the zero-padded second block
        indptr, indices, blocks, shape, A = _case(1024, 6, per_row)
        B = synth.dense_features(shape[1], N, 1)
        a = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, dtype, cuda_device)
        Bd = torch.from_numpy(B).to(cuda_device).to(tdt)
        C = bsr.spmm_bsr8(a, Bd).cpu().numpy()
        want = A @ B.astype(np.float64)
        scale = np.abs(want).max()
        assert np.abs(C - want).max() <= 1e-2 * scale
        Ar = sp.bsr_matrix((a.blocks.float().cpu().numpy().astype(np.float64), indices, indptr), shape=shape)
        want_r = Ar @ Bd.float().cpu().numpy().astype(np.float64)
        np.testing.assert_allclose(C, want_r, rtol=1e-5, atol=1e-4)


def test_empty_block_rows_and_row_ranges(cuda_device):
    import torch
    indptr, indices, blocks, shape, _ = _case(1024, 7)
    keep = np.ones(len(indices), dtype=bool)
    for I in (0, 17, 127):
        keep[indptr[I]:indptr[I + 1]] = False
    counts = np.diff(indptr).copy()
    counts[[0, 17, 127]] = 0
    indptr2 = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    A = sp.bsr_matrix((blocks[keep].astype(np.float64), indices[keep], indptr2), shape=shape)
    B = synth.dense_features(shape[1], 64, 2)
    a = bsr.DeviceBsr8.from_arrays(indptr2, indices[keep], blocks[keep], shape, "float32", cuda_device)
    Bd = torch.from_numpy(B).to(cuda_device)
    C = bsr.spmm_bsr8(a, Bd).cpu().numpy()
    want = A @ B.astype(np.float64)
    np.testing.assert_allclose(C, want, rtol=1e-5, atol=1e-4)
    assert not C[0:8].any() and not C[17 * 8:18 * 8].any()
    part = bsr.spmm_bsr8(a, Bd, block_row_range=(40, 100)).cpu().numpy()
    np.testing.assert_allclose(part, want[320:800], rtol=1e-5, atol=1e-4)


def test_bench_bsrmm_dropin_with_32x32_fp16_blocks(cuda_device):
    """The reference's call: scipy BSR with 32x32 fp16 blocks and a half-precision x."""
    import torch
    from liteform_ae_b200.format_matrix_market import MTX
    from liteform_ae_b200 import format_algos as fa
    csr = synth.zipf_rows(M=1024, seed=3)
    g = MTX.from_csr(csr.indptr, csr.indices, np.ones(csr.nnz), csr.shape)
    bsr_mat = g.tobsr_with_padding(shape=(1024, 1024), blocksize=(32, 32))
    x = torch.rand(1024, 64).half()
    ms = fa.bench_bsrmm(bsr_mat, x, block_size=32, device=cuda_device, warmup=1, repeat=3)
    assert ms > 0
    a = bsr.DeviceBsr8.from_scipy(bsr_mat, device=cuda_device)
    C = bsr.spmm_bsr8(a, x.to(cuda_device)).cpu().numpy()
    want = g.coo_mtx.tocsr() @ x.float().numpy().astype(np.float64)
    np.testing.assert_allclose(C, want, rtol=1e-4, atol=1e-3)


def test_unsupported_shapes_are_rejected(cuda_device):
    import torch
    indptr, indices, blocks, shape, _ = _case(256, 1)
    a = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, "float32", cuda_device)
    with pytest.raises(Exception, match="multiples of 4"):
        bsr.spmm_bsr8(a, torch.zeros((shape[1], 6), device=cuda_device))
