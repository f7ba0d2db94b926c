"""Tuning knobs select differently compiled kernels; none of them may change the result."""
import itertools

import numpy as np
import pytest

from oracle import hyb_oracle as ho
from liteform_ae_b200 import _cabi, bsr, hyb, synth

pytestmark = pytest.mark.gpu

DEFAULT_GATHER_RING = 16  # the library's initial value of LF_OPT_SPMM_GATHER_RING


@pytest.fixture
def restore_defaults():
    yield
    lib = _cabi.load()
    lib.lf_set_option(_cabi.LF_OPT_SPMM_CACHE_POLICY, 1)
    lib.lf_set_option(_cabi.LF_OPT_SPMM_MIN_BLOCKS, 3)
    lib.lf_set_option(_cabi.LF_OPT_SPMM_SLOTS_PER_GROUP, 0)
    lib.lf_bsr_set_tuning(0, 0, 0)
    lib.lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, 0)
    lib.lf_set_option(_cabi.LF_OPT_BSR_TILE_ORDER, 0)
    lib.lf_set_option(_cabi.LF_OPT_SPMM_TILE_SEGMENTS, 0)
    lib.lf_set_option(_cabi.LF_OPT_BSR_PIPE_SHAPE, 0)
    lib.lf_set_option(_cabi.LF_OPT_BSR_PIPE_3D, 1)
    lib.lf_set_option(_cabi.LF_OPT_BSR_UMMA_PRODUCER, 0)
    lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, DEFAULT_GATHER_RING)
    lib.lf_set_option(_cabi.LF_OPT_BSR_BLOCK_WARPS, 0)
    lib.lf_set_option(_cabi.LF_OPT_SPMM_RING_MIN_SLOTS, 1 << 20)


def test_every_spmm_variant_gives_the_same_product(cuda_device, restore_defaults):
    import torch
    lib = _cabi.load()
    csr = synth.skewed_rows(M=4096, seed=5, heavy_rows=6, heavy_len=3000)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    fmt = hyb.build_hyb_device(d, [[1, 2, 4, 8, 16]], with_mask=False)
    for N in (32, 128, 512):
        B = synth.dense_features(4096, N, 2)
        Bd = torch.from_numpy(B).to(cuda_device)
        want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, B.astype(np.float64))
        for pol, minb, slots, segs in itertools.product((0, 1), (2, 3, 4), (0, 8, 64, 4096), (0, 1, 7, 64)):
            # the occupancy knob belongs to the register kernel; the ring kernel takes the other three
            assert lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, 0 if minb != 3 else 16) == 0
            assert lib.lf_set_option(_cabi.LF_OPT_SPMM_CACHE_POLICY, pol) == 0
            assert lib.lf_set_option(_cabi.LF_OPT_SPMM_MIN_BLOCKS, minb) == 0
            assert lib.lf_set_option(_cabi.LF_OPT_SPMM_SLOTS_PER_GROUP, slots) == 0
            assert lib.lf_set_option(_cabi.LF_OPT_SPMM_TILE_SEGMENTS, segs) == 0
            C = hyb.spmm_hyb(fmt, Bd).cpu().numpy()
            np.testing.assert_allclose(C, want, rtol=1e-5, atol=1e-4, err_msg=f"{N} {pol} {minb} {slots} {segs}")
    assert lib.lf_set_option(_cabi.LF_OPT_SPMM_CACHE_POLICY, 2) == _cabi.LF_ERR_INVALID_ARGUMENT
    assert lib.lf_set_option(_cabi.LF_OPT_SPMM_MIN_BLOCKS, 7) == _cabi.LF_ERR_INVALID_ARGUMENT
    assert lib.lf_set_option(99, 1) == _cabi.LF_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("parts", [1, 3])
def test_gather_ring_adds_up_in_the_same_order_as_the_register_kernel(cuda_device, restore_defaults, parts):
    """Gathers that land in a shared-memory ring (cp.async, 16 rows ahead) instead of registers:
    the slots of a thread group are added in the same order, so rows that one group owns are
    bit-identical; rows reduced by atomics over several groups agree to rounding."""
    import torch
    lib = _cabi.load()
    csr = synth.skewed_rows(M=6000, seed=8, heavy_rows=5, heavy_len=2500)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    widths = [[1, 2, 4, 8, 16, 64]] if parts == 1 else [[1, 4, 32], [2, 8], [1, 2, 4, 8, 16]]
    fmt = hyb.build_hyb_device(d, widths, with_mask=False)
    for N in (100, 128, 256, 320, 512):
        B = synth.dense_features(csr.shape[1], N, 3)
        Bd = torch.from_numpy(B).to(cuda_device)
        want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, B.astype(np.float64))
        for slots, pol in itertools.product((0, 8, 40, 4096), (0, 1)):
            assert lib.lf_set_option(_cabi.LF_OPT_SPMM_SLOTS_PER_GROUP, slots) == 0
            assert lib.lf_set_option(_cabi.LF_OPT_SPMM_CACHE_POLICY, pol) == 0
            assert lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, 0) == 0
            base = hyb.spmm_hyb(fmt, Bd)
            for depth in (16,):
                assert lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, depth) == 0
                C = torch.full((csr.shape[0], N), float("nan"), device=cuda_device)
                hyb.spmm_hyb(fmt, Bd, out=C)
                got = C.cpu().numpy()
                np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-4, err_msg=f"{N} {slots} {pol} {depth}")
                if parts == 1:
                    short = np.diff(csr.indptr) <= 64     # one ELL row, one group, no atomics
                    assert np.array_equal(got[short], base.cpu().numpy()[short])
    assert lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, 8) == _cabi.LF_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("parts", [1, 3])
def test_gather_ring_with_rows_narrower_than_a_warp(cuda_device, restore_defaults, parts):
    """Up to 64 float32 / 128 bf16 features a warp of the ring kernel takes 2 or 4 slots per step and adds
    the partial sums at the flush; buckets narrower than that run the register kernel in a second launch."""
    import torch
    lib = _cabi.load()
    assert lib.lf_set_option(_cabi.LF_OPT_SPMM_RING_MIN_SLOTS, 0) == 0    # small matrices take the ring form too
    csr = synth.skewed_rows(M=6000, seed=8, heavy_rows=5, heavy_len=2500)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    for widths in ([[1, 2, 4, 8, 16, 64]], [[4, 32]], [[1]], [[2, 16]]) if parts == 1 else ([[1, 4, 32], [2, 8], [1, 2, 4, 8, 16]],):
        fmt = hyb.build_hyb_device(d, widths, with_mask=False)
        for N in (4, 20, 32, 48, 64):
            B = synth.dense_features(csr.shape[1], N, 3)
            Bd = torch.from_numpy(B).to(cuda_device)
            want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, B.astype(np.float64))
            for slots, depth in itertools.product((0, 8, 40, 4096), (0, 16)):
                assert lib.lf_set_option(_cabi.LF_OPT_SPMM_SLOTS_PER_GROUP, slots) == 0
                assert lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, depth) == 0
                C = torch.full((csr.shape[0], N), float("nan"), device=cuda_device)
                hyb.spmm_hyb(fmt, Bd, out=C)
                np.testing.assert_allclose(C.cpu().numpy(), want, rtol=1e-5, atol=1e-4, err_msg=f"{widths} {N} {slots} {depth}")
                C.fill_(1.0)
                hyb.spmm_hyb(fmt, Bd, out=C, accumulate=True)
                np.testing.assert_allclose(C.cpu().numpy(), want + 1.0, rtol=1e-5, atol=2e-4, err_msg=f"acc {widths} {N} {slots} {depth}")
        for N in (64, 128):      # bf16 features: 8 per lane
            B = synth.dense_features(csr.shape[1], N, 4)
            B16 = torch.from_numpy(B).to(cuda_device).to(torch.bfloat16)
            want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape,
                                     B16.float().cpu().numpy().astype(np.float64))
            for depth in (0, 16):
                assert lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, depth) == 0
                np.testing.assert_allclose(hyb.spmm_hyb(fmt, B16).cpu().numpy(), want, rtol=1e-5, atol=1e-4)


@pytest.mark.parametrize("N", [32, 64, 128, 320])
def test_ring_kernels_with_strided_operands(cuda_device, restore_defaults, N):
    """B and C as column windows of wider matrices (leading dimensions larger than N, bases off the
    row start): the ring kernels multiply the column by the row pitch and must leave the rest of C alone."""
    import torch
    lib = _cabi.load()
    assert lib.lf_set_option(_cabi.LF_OPT_SPMM_RING_MIN_SLOTS, 0) == 0
    csr = synth.skewed_rows(M=5000, seed=12, heavy_rows=3, heavy_len=1800)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    fmt = hyb.build_hyb_device(d, [[1, 2, 4, 8, 32]], with_mask=False)
    B = synth.dense_features(csr.shape[1], N, 7)
    want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, B.astype(np.float64))
    Bbig = torch.zeros((csr.shape[1], N + 40), device=cuda_device)
    Bbig[:, 8:8 + N] = torch.from_numpy(B).to(cuda_device)
    for depth in (0, 16):
        assert lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, depth) == 0
        Cbig = torch.full((csr.shape[0], N + 24), -1.0, device=cuda_device)
        hyb.spmm_hyb(fmt, Bbig[:, 8:8 + N], out=Cbig[:, 4:4 + N])
        got = Cbig.cpu().numpy()
        np.testing.assert_allclose(got[:, 4:4 + N], want, rtol=1e-5, atol=1e-4)
        assert (got[:, :4] == -1).all() and (got[:, 4 + N:] == -1).all()
        C2 = torch.full((csr.shape[0], N + 24), -1.0, device=cuda_device)
        hyb.spmm_csr(d, Bbig[:, 8:8 + N], out=C2[:, 4:4 + N])
        got = C2.cpu().numpy()
        np.testing.assert_allclose(got[:, 4:4 + N], want, rtol=1e-5, atol=1e-4)
        assert (got[:, :4] == -1).all() and (got[:, 4 + N:] == -1).all()


@pytest.mark.parametrize("N", [100, 128, 384])
def test_csr_product_with_and_without_the_gather_ring(cuda_device, restore_defaults, N):
    """lf_spmm_csr_f32 has the same two forms; rows that one thread group owns are bit-identical."""
    import torch
    lib = _cabi.load()
    csr = synth.skewed_rows(M=6000, seed=9, heavy_rows=4, heavy_len=2000)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    B = synth.dense_features(csr.shape[1], N, 6)
    Bd = torch.from_numpy(B).to(cuda_device)
    want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, B.astype(np.float64))
    got = {}
    for depth in (0, 16):
        assert lib.lf_set_option(_cabi.LF_OPT_SPMM_GATHER_RING, depth) == 0
        for rr in ((0, csr.shape[0]), (123, 4567)):
            C = torch.full((rr[1] - rr[0], N), float("nan"), device=cuda_device)
            hyb.spmm_csr(d, Bd, out=C, row_range=rr)
            got[depth, rr] = C.cpu().numpy()
            np.testing.assert_allclose(got[depth, rr], want[rr[0]:rr[1]], rtol=1e-5, atol=1e-4)
    full = (0, csr.shape[0])
    same = (got[0, full] == got[16, full]).all(axis=1)
    assert same.mean() > 0.9     # all but the rows cut by a group boundary (reduced by atomics in any order)


def test_every_block_kernel_variant_gives_the_same_product(cuda_device, restore_defaults):
    import scipy.sparse as sp
    import torch
    lib = _cabi.load()
    indptr, indices, blocks, shape = synth.banded_blocks(M=2048, seed=3, per_block_row=7, half_band=50)
    A = sp.bsr_matrix((blocks.astype(np.float64), indices, indptr), shape=shape)
    a32 = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, "float32", cuda_device)
    a16 = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, "bfloat16", cuda_device)
    A16 = sp.bsr_matrix((a16.blocks.float().cpu().numpy().astype(np.float64), indices, indptr), shape=shape)
    for N in (64, 136, 256):
        B = synth.dense_features(shape[1], N, 4)
        Bd = torch.from_numpy(B).to(cuda_device)
        B16 = Bd.to(torch.bfloat16)
        want = A @ B.astype(np.float64)
        want16 = A16 @ B16.float().cpu().numpy().astype(np.float64)
        for engine, units, stages, rpw in itertools.product((1, 2, 3), (0, 1, 2), (0, 3, 4), (0, 1, 5, 31)):
            assert lib.lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, engine) == 0
            assert lib.lf_bsr_set_tuning(units, stages, rpw) == 0
            np.testing.assert_allclose(bsr.spmm_bsr8(a32, Bd).cpu().numpy(), want, rtol=1e-5, atol=1e-4)
            np.testing.assert_allclose(bsr.spmm_bsr8(a16, B16).cpu().numpy(), want16, rtol=1e-5, atol=1e-4)
        assert lib.lf_bsr_copy_status(None) == 0   # no warp gave up waiting for a bulk copy
        for engine, order in itertools.product((1, 2, 3), (0, 1, 2)):
            assert lib.lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, engine) == 0
            assert lib.lf_set_option(_cabi.LF_OPT_BSR_TILE_ORDER, order) == 0
            assert lib.lf_bsr_set_tuning(2, 0, 0) == 0
            np.testing.assert_allclose(bsr.spmm_bsr8(a32, Bd).cpu().numpy(), want, rtol=1e-5, atol=1e-4)
        assert lib.lf_set_option(_cabi.LF_OPT_BSR_TILE_ORDER, 0) == 0
        assert lib.lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, 1) == 0
        assert lib.lf_bsr_set_tuning(0, 0, 0) == 0
        for warps in (1, 3, 4, 8):      # thread blocks of fewer warps: same warp-private rings, same result
            assert lib.lf_set_option(_cabi.LF_OPT_BSR_BLOCK_WARPS, warps) == 0
            np.testing.assert_allclose(bsr.spmm_bsr8(a32, Bd).cpu().numpy(), want, rtol=1e-5, atol=1e-4)
            np.testing.assert_allclose(bsr.spmm_bsr8(a16, B16).cpu().numpy(), want16, rtol=1e-5, atol=1e-4)
        assert lib.lf_set_option(_cabi.LF_OPT_BSR_BLOCK_WARPS, 0) == 0
    assert lib.lf_bsr_set_tuning(3, 0, 0) == _cabi.LF_ERR_INVALID_ARGUMENT
    assert lib.lf_set_option(_cabi.LF_OPT_BSR_BLOCK_WARPS, 9) == _cabi.LF_ERR_INVALID_ARGUMENT
    assert lib.lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, 6) == _cabi.LF_ERR_INVALID_ARGUMENT


@pytest.mark.parametrize("per_row", [8, 5, 1, 19])
def test_thread_block_pipeline_gives_the_same_product(cuda_device, restore_defaults, per_row):
    """Copy engines 4 (producer warp + tiled bulk copies + consumer warps with mma.sync) and 5 (the
    same copies feeding tcgen05.mma, accumulators in tensor memory; 16-bit inputs) in every ring shape, with
    one 3-D copy per block and with one 2-D copy per feature slice, float32 and both 16-bit types,
    feature widths that fill, underfill and overflow the 128- / 256-feature tiles, block rows
    with 1, 5, 8 and 19 blocks (odd counts pair the last block with zeros; 19 spans several
    stages), empty block rows and row ranges."""
    import scipy.sparse as sp
    import torch
    lib = _cabi.load()
    indptr, indices, blocks, shape = synth.banded_blocks(M=4096, seed=11, per_block_row=per_row, half_band=60)
    indptr = indptr.astype(np.int64)
    keep = np.ones(len(indices), dtype=bool)
    counts = np.diff(indptr).copy()
    for I in (0, 3, 40, 511):                 # some block rows lose all their blocks
        keep[indptr[I]:indptr[I + 1]] = False
        counts[I] = 0
    indptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int64)
    indices, blocks = indices[keep], blocks[keep]
    A = sp.bsr_matrix((blocks.astype(np.float64), indices, indptr), shape=shape)
    a32 = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, "float32", cuda_device)
    assert lib.lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, 4) == 0
    for N in (40, 64, 128, 136, 160, 256, 384, 512):
        B = synth.dense_features(shape[1], N, 6)
        Bd = torch.from_numpy(B).to(cuda_device)
        want = A @ B.astype(np.float64)
        for shape_code, three_d, rpc in itertools.product((0, 43, 83, 26), (1, 0), (0, 7)):
            assert lib.lf_set_option(_cabi.LF_OPT_BSR_PIPE_SHAPE, shape_code) == 0
            assert lib.lf_set_option(_cabi.LF_OPT_BSR_PIPE_3D, three_d) == 0
            assert lib.lf_bsr_set_tuning(0, 0, rpc) == 0
            C = torch.full((shape[0], N), float("nan"), device=cuda_device)
            bsr.spmm_bsr8(a32, Bd, out=C)
            np.testing.assert_allclose(C.cpu().numpy(), want, rtol=1e-5, atol=1e-4, err_msg=f"f32 {N} {shape_code} {three_d} {rpc}")
        part = bsr.spmm_bsr8(a32, Bd, block_row_range=(37, 300)).cpu().numpy()
        np.testing.assert_allclose(part, want[37 * 8:300 * 8], rtol=1e-5, atol=1e-4)
        for dtype in ("bfloat16", "float16"):
            tdt = getattr(torch, dtype)
            a16 = bsr.DeviceBsr8.from_arrays(indptr, indices, blocks, shape, dtype, cuda_device)
            A16 = sp.bsr_matrix((a16.blocks.float().cpu().numpy().astype(np.float64), indices, indptr), shape=shape)
            B16 = Bd.to(tdt)
            want16 = A16 @ B16.float().cpu().numpy().astype(np.float64)
            for engine, shape_code, three_d in itertools.product((4, 5), (0, 43, 83, 46, 86, 24), (1, 0, 2, 4)):
                # engine 5: three_d doubles as the producer choice (1 / 0: tiled copies, 3-D / 2-D; 2 / 4: cp.async warps)
                if engine == 4 and three_d > 1:
                    continue
                assert lib.lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, engine) == 0
                assert lib.lf_set_option(_cabi.LF_OPT_BSR_PIPE_SHAPE, shape_code) == 0
                assert lib.lf_set_option(_cabi.LF_OPT_BSR_PIPE_3D, min(three_d, 1)) == 0
                assert lib.lf_set_option(_cabi.LF_OPT_BSR_UMMA_PRODUCER, three_d if three_d > 1 else 0) == 0
                C = torch.full((shape[0], N), float("nan"), device=cuda_device)
                bsr.spmm_bsr8(a16, B16, out=C)
                np.testing.assert_allclose(C.cpu().numpy(), want16, rtol=1e-5, atol=1e-4,
                                           err_msg=f"{dtype} {N} engine {engine} {shape_code} {three_d}")
            assert lib.lf_set_option(_cabi.LF_OPT_BSR_COPY_ENGINE, 4) == 0
    assert lib.lf_bsr_copy_status(None) == 0   # no thread block gave up waiting for a copy
