"""CSR -> 8x8 blocks on the device (lf_bsr8_plan / lf_bsr8_fill) vs SciPy's own conversion, which is
what the reference calls (MTX.tobsr_with_padding -> scipy.sparse.bsr_matrix).  Integer arrays and
float32 tiles must be bit-exact; 16-bit tiles must equal the round-to-nearest-even cast."""
import numpy as np
import pytest
import scipy.sparse as sp

from liteform_ae_b200 import bsr, hyb, synth
from liteform_ae_b200.format_matrix_market import MTX

pytestmark = pytest.mark.gpu


def _scipy_bsr8(csr, shape8):
    m = sp.csr_matrix((csr.data, csr.indices, csr.indptr), shape=csr.shape)
    m.resize(shape8)
    b = m.tobsr(blocksize=(8, 8))
    b.sort_indices()
    return b


def _random_csr(M, K, seed, density, empty_rows=True):
    rng = np.random.default_rng(seed)
    m = sp.random(M, K, density=density, random_state=rng, format="csr", dtype=np.float32)
    m.data = rng.uniform(0.5, 1.5, m.nnz).astype(np.float32)   # no explicit zeros
    if empty_rows and M > 16:
        lil = m.tolil()
        lil[3, :] = 0
        lil[8:16, :] = 0            # a block row without any block
        m = lil.tocsr()
        m.eliminate_zeros()
    m.sort_indices()
    return synth.Csr(m.indptr.astype(np.int64), m.indices.astype(np.int32), m.data.astype(np.float32), m.shape, "random")


CASES = [(64, 64, 0.2), (61, 75, 0.1), (7, 5, 0.5), (1, 1, 1.0), (1000, 333, 0.02), (4096, 4096, 0.003), (257, 2049, 0.3)]


@pytest.mark.parametrize("M,K,density", CASES)
def test_device_blocks_equal_scipy(cuda_device, M, K, density):
    csr = _random_csr(M, K, M * 31 + K, density)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    a = bsr.DeviceBsr8.from_csr_device(d, "float32")
    shape8 = (-(-M // 8) * 8, -(-K // 8) * 8)
    want = _scipy_bsr8(csr, shape8)
    assert a.shape == shape8
    np.testing.assert_array_equal(a.indptr.cpu().numpy(), want.indptr.astype(np.int64))
    np.testing.assert_array_equal(a.indices.cpu().numpy(), want.indices.astype(np.int32))
    np.testing.assert_array_equal(a.blocks.cpu().numpy(), want.data.reshape(-1, 8, 8))


@pytest.mark.parametrize("dtype", ["bfloat16", "float16"])
def test_16bit_tiles_are_the_rounded_float32_tiles(cuda_device, dtype):
    import torch
    csr = _random_csr(520, 300, 5, 0.05)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    a32 = bsr.DeviceBsr8.from_csr_device(d, "float32")
    a16 = bsr.DeviceBsr8.from_csr_device(d, dtype)
    assert torch.equal(a16.indptr, a32.indptr) and torch.equal(a16.indices, a32.indices)
    assert torch.equal(a16.blocks, a32.blocks.to(getattr(torch, dtype)))


def test_pattern_only_matrix_and_padded_shape(cuda_device):
    import torch
    csr = _random_csr(100, 90, 9, 0.1)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, None, csr.shape, cuda_device)   # data = None: all ones
    a = bsr.DeviceBsr8.from_csr_device(d, "float32", padded_shape=(128, 128))
    ones = synth.Csr(csr.indptr, csr.indices, np.ones_like(csr.data), csr.shape, "ones")
    want = _scipy_bsr8(ones, (128, 128))
    assert a.shape == (128, 128)
    np.testing.assert_array_equal(a.indptr.cpu().numpy(), want.indptr.astype(np.int64))
    np.testing.assert_array_equal(a.indices.cpu().numpy(), want.indices.astype(np.int32))
    np.testing.assert_array_equal(a.blocks.cpu().numpy(), want.data.reshape(-1, 8, 8))
    # and the product through the block kernel equals the CSR product
    B = synth.dense_features(128, 64, 3)
    C = bsr.spmm_bsr8(a, torch.from_numpy(B).to(cuda_device)).cpu().numpy()
    ref = sp.csr_matrix((ones.data, ones.indices, ones.indptr), shape=(100, 90)).astype(np.float64) @ B[:90].astype(np.float64)
    np.testing.assert_allclose(C[:100], ref, rtol=1e-5, atol=1e-4)
    assert not C[100:].any()


def test_mtx_tobsr_device_matches_the_host_conversion(cuda_device):
    csr = _random_csr(200, 200, 11, 0.05, empty_rows=False)
    g = MTX.from_csr(csr.indptr, csr.indices, csr.data, csr.shape, "t")
    host = g.tobsr_with_padding(shape=(224, 224), blocksize=(32, 32))          # what the reference builds
    a_host = bsr.DeviceBsr8.from_scipy(host, device=cuda_device)                # re-blocked on the host
    a_dev = g.tobsr_device(shape=(224, 224), dtype="float16", device=cuda_device)
    # the host path keeps only 8x8 tiles with entries, as the device path does
    np.testing.assert_array_equal(a_dev.indptr.cpu().numpy(), a_host.indptr.cpu().numpy())
    np.testing.assert_array_equal(a_dev.indices.cpu().numpy(), a_host.indices.cpu().numpy())
    np.testing.assert_array_equal(a_dev.blocks.float().cpu().numpy(), a_host.blocks.float().cpu().numpy())


def test_full_size_block_matrix_round_trip(cuda_device):
    """BSR -> CSR on the host -> BSR on the device gives the blocks back (banded benchmark pattern)."""
    indptr, indices, blocks, shape = synth.banded_blocks(M=1 << 15, seed=4)
    csr = synth.bsr_to_csr(indptr, indices, blocks, shape)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    a = bsr.DeviceBsr8.from_csr_device(d, "float32")
    np.testing.assert_array_equal(a.indptr.cpu().numpy(), np.asarray(indptr, dtype=np.int64))
    np.testing.assert_array_equal(a.indices.cpu().numpy(), np.asarray(indices, dtype=np.int32))
    np.testing.assert_array_equal(a.blocks.cpu().numpy(), blocks)


def _scipy_split8(m):
    """The host route the device split replaces: float32 copy -> CSR -> explicit zeros dropped -> 8x8 blocks."""
    R, Cb = m.blocksize
    m32 = sp.bsr_matrix((m.data.astype(np.float32), m.indices, m.indptr), shape=m.shape, blocksize=(R, Cb))
    csr = m32.tocsr()
    csr.eliminate_zeros()
    out = sp.bsr_matrix(csr, blocksize=(8, 8))
    out.sort_indices()
    return out


@pytest.mark.parametrize("blocksize", [(32, 32), (16, 24), (8, 8)])
@pytest.mark.parametrize("in_dtype", [np.float32, np.float16])
def test_coarse_blocks_are_cut_into_tiles_on_the_device(cuda_device, blocksize, in_dtype):
    """lf_bsr_split8_plan / lf_bsr_split8_fill vs SciPy: tiles that hold only zeros (padding inside
    coarse blocks, explicit zeros, -0.0) are dropped, block columns come out sorted, values are
    copied bit for bit."""
    R, Cb = blocksize
    rng = np.random.default_rng(R * 100 + Cb)
    Mb, Kb, per_row = 37, 29, 5
    indptr = np.arange(Mb + 1, dtype=np.int32) * per_row
    cols = np.stack([rng.permutation(Kb)[:per_row] for _ in range(Mb)])        # NOT sorted inside a block row
    data = rng.uniform(-1, 1, size=(Mb * per_row, R, Cb)).astype(np.float32)
    data[rng.random(data.shape) < 0.93] = 0.0                                   # most 8x8 tiles end up empty
    data[0, :8, :8] = 0.0
    data[0, 0, 0] = -0.0                                                        # a tile of zeros only (one negative)
    data[1, 8 % R:8 % R + 8, :8] = 0.0
    m = sp.bsr_matrix((data, cols.reshape(-1), indptr), shape=(Mb * R, Kb * Cb), blocksize=(R, Cb))
    if in_dtype != np.float32:       # SciPy builds no float16 matrix; narrow the block array afterwards
        m.data = m.data.astype(in_dtype)
    want = _scipy_split8(m)
    for out_dtype in ("float32", "float16", "bfloat16"):
        a = bsr.DeviceBsr8.from_scipy(m, dtype=out_dtype, device=cuda_device)
        assert a.shape == m.shape
        np.testing.assert_array_equal(a.indptr.cpu().numpy(), want.indptr.astype(np.int64))
        np.testing.assert_array_equal(a.indices.cpu().numpy(), want.indices.astype(np.int32))
        import torch
        ref = torch.from_numpy(want.data.astype(np.float32)).to(getattr(torch, out_dtype))
        assert torch.equal(a.blocks.cpu().view(torch.int16 if out_dtype != "float32" else torch.int32),
                           ref.view(torch.int16 if out_dtype != "float32" else torch.int32))


def test_coarse_block_matrix_without_blocks(cuda_device):
    m = sp.bsr_matrix((np.zeros((0, 32, 32), dtype=np.float32), np.zeros(0, dtype=np.int32), np.zeros(5, dtype=np.int32)),
                      shape=(128, 96), blocksize=(32, 32))
    a = bsr.DeviceBsr8.from_scipy(m, device=cuda_device)
    assert a.num_blocks == 0 and a.indptr.numel() == 17 and not a.indptr.any()
