"""Error behaviour of the C ABI: bad arguments come back as negative status codes with a message,
nothing is thrown and nothing faults (every check happens on the host before a launch)."""
import ctypes as C

import numpy as np
import pytest

from liteform_ae_b200 import _cabi, hyb, synth

pytestmark = pytest.mark.gpu


def test_status_codes_and_messages(cuda_device):
    import torch
    lib = _cabi.load()
    csr = synth.zipf_rows(M=512, seed=1)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    stats = torch.empty(33, dtype=torch.int64, device=cuda_device)
    hist = torch.empty(2048, dtype=torch.int64, device=cuda_device)
    small = torch.empty(16, dtype=torch.uint8, device=cuda_device)
    rc = lib.lf_hyb_stats(d.indptr.data_ptr(), d.indices.data_ptr(), 512, 512, 1, stats.data_ptr(), hist.data_ptr(),
                          small.data_ptr(), small.numel(), 0)
    assert rc == _cabi.LF_ERR_WORKSPACE_TOO_SMALL and b"workspace" in lib.lf_last_error()
    rc = lib.lf_hyb_stats(0, d.indices.data_ptr(), 512, 512, 1, stats.data_ptr(), hist.data_ptr(), small.data_ptr(), 16, 0)
    assert rc == _cabi.LF_ERR_INVALID_ARGUMENT
    rc = lib.lf_hyb_stats(d.indptr.data_ptr(), d.indices.data_ptr(), 512, 512, 0, stats.data_ptr(), hist.data_ptr(),
                          small.data_ptr(), 16, 0)
    assert rc == _cabi.LF_ERR_INVALID_ARGUMENT and b"num_parts" in lib.lf_last_error()

    fmt = hyb.build_hyb_device(d, [[1, 2, 4, 8, 16, 32]])
    B = torch.zeros((512, 32), device=cuda_device)
    Cout = torch.zeros((512, 32), device=cuda_device)
    s = fmt.c_struct()
    assert lib.lf_spmm_hyb_f32(C.byref(s), B.data_ptr(), 16, Cout.data_ptr(), 32, 32, 0, 0) == _cabi.LF_ERR_INVALID_ARGUMENT
    assert b"leading" in lib.lf_last_error()
    assert lib.lf_spmm_hyb_f32(C.byref(s), B.data_ptr(), 32, Cout.data_ptr(), 32, 32, 9, 0) == _cabi.LF_ERR_INVALID_ARGUMENT
    assert lib.lf_spmm_hyb_f32(C.byref(s), 0, 32, Cout.data_ptr(), 32, 32, 0, 0) == _cabi.LF_ERR_INVALID_ARGUMENT
    assert lib.lf_spmm_hyb_f32(None, B.data_ptr(), 32, Cout.data_ptr(), 32, 32, 0, 0) == _cabi.LF_ERR_INVALID_ARGUMENT
    bad = fmt.c_struct()
    bad.row_end = 10 ** 9
    assert lib.lf_spmm_hyb_f32(C.byref(bad), B.data_ptr(), 32, Cout.data_ptr(), 32, 32, 0, 0) == _cabi.LF_ERR_INVALID_ARGUMENT
    with pytest.raises(_cabi.LiteformError):
        hyb.build_hyb_device(d, [[1, 2, 4]], row_range=(5, 10 ** 7))
    assert lib.lf_shard_rows(d.indptr.data_ptr(), 512, 0, stats.data_ptr(), 0) == _cabi.LF_ERR_INVALID_ARGUMENT


def test_empty_inputs(cuda_device):
    """No rows, no entries, empty row range: every call succeeds and writes nothing out of range."""
    import torch
    empty = synth.Csr(np.zeros(5, dtype=np.int64), np.zeros(0, dtype=np.int32), np.zeros(0, dtype=np.float32), (4, 6))
    d = hyb.DeviceCsr.from_host(empty.indptr, empty.indices, empty.data, empty.shape, cuda_device)
    stats, hist = hyb.hyb_stats(d, 2)
    assert not stats.any() and not hist.any()
    fmt = hyb.build_hyb_device(d, [[], []])
    assert fmt.num_zero_rows == 4 and fmt.total_slots == 0
    B = torch.randn((6, 8), device=cuda_device)
    Cout = torch.full((4, 8), 3.0, device=cuda_device)
    hyb.spmm_hyb(fmt, B, out=Cout)
    assert not Cout.any()
    csr = synth.zipf_rows(M=256, seed=2)
    d2 = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    part = hyb.build_hyb_device(d2, [[1, 2, 4, 8, 16, 32, 64]], row_range=(100, 100))
    assert hyb.spmm_hyb(part, torch.randn((256, 8), device=cuda_device)).shape == (0, 8)
    assert hyb.spmm_csr(d2, torch.randn((256, 8), device=cuda_device), row_range=(7, 7)).shape == (0, 8)


def test_malformed_matrices_are_reported_not_dereferenced(cuda_device):
    """Column indices outside the matrix, unsorted rows and broken row pointers: lf_csr_validate
    names the defect, the builder kernels skip the bad entries (no access outside their arrays)
    and lf_hyb_plan returns an error instead of a format."""
    import torch
    lib = _cabi.load()
    indptr = np.array([0, 3, 5, 9], dtype=np.int64)
    good = np.array([0, 2, 5, 1, 3, 0, 1, 4, 7], dtype=np.int32)
    shape = (3, 8)
    hyb.DeviceCsr.from_host(indptr, good, None, shape, cuda_device)                      # passes
    for bad_idx, what in ((np.array([0, 2, 5, 1, 3, 0, 1, 4, 8], dtype=np.int32), "outside"),
                          (np.array([0, 2, 5, 1, -3, 0, 1, 4, 7], dtype=np.int32), "outside"),
                          (np.array([0, 5, 2, 1, 3, 0, 1, 4, 7], dtype=np.int32), "ascending"),
                          (np.array([0, 2, 2, 1, 3, 0, 1, 4, 7], dtype=np.int32), "ascending")):
        with pytest.raises(ValueError, match=what):
            hyb.DeviceCsr.from_host(indptr, bad_idx, None, shape, cuda_device)
    with pytest.raises(ValueError, match="row pointers"):
        hyb.DeviceCsr.from_host(np.array([0, 5, 3, 9], dtype=np.int64), good, None, shape, cuda_device)
    with pytest.raises(ValueError, match="row pointers"):
        hyb.DeviceCsr.from_host(np.array([0, 3, 5, 8], dtype=np.int64), good, None, shape, cuda_device)
    with pytest.raises(ValueError, match="2\\^31"):
        hyb.DeviceCsr.from_host(indptr, good.astype(np.int64) + (1 << 32), None, shape, cuda_device)
    # the kernels themselves, fed the out-of-range matrix without validation: statistics complete
    # (bad entries skipped), the plan refuses
    bad = np.array([0, 2, 5, 1, 3, 0, 1, 4, 1 << 20], dtype=np.int32)
    d = hyb.DeviceCsr.from_host(indptr, bad, None, shape, cuda_device, validate=False)
    for P in (1, 2):
        stats, hist = hyb.hyb_stats(d, P)
        assert stats[..., 2].sum() >= 3
    with pytest.raises(_cabi.LiteformError, match="outside"):
        hyb.build_hyb_device(d, [[1, 2, 4], [1, 2, 4]])
    # argument checks of the statistics call come before any launch: the outputs stay untouched
    stats_d = torch.full((33,), -7, dtype=torch.int64, device=cuda_device)
    hist_d = torch.full((2048,), -7, dtype=torch.int64, device=cuda_device)
    ws = torch.empty(lib.lf_hyb_stats_workspace_bytes(3, 8, 1), dtype=torch.uint8, device=cuda_device)
    rc = lib.lf_hyb_stats(d.indptr.data_ptr(), d.indices.data_ptr(), 3, 8, 9, stats_d.data_ptr(), hist_d.data_ptr(),
                          ws.data_ptr(), ws.numel(), 0)
    assert rc == _cabi.LF_ERR_INVALID_ARGUMENT
    torch.cuda.synchronize()
    assert bool((stats_d == -7).all()) and bool((hist_d == -7).all())


def test_block_matrix_without_blocks_gives_zero(cuda_device):
    import torch
    from liteform_ae_b200 import bsr
    a = bsr.DeviceBsr8(torch.zeros(5, dtype=torch.int64, device=cuda_device),
                       torch.zeros(0, dtype=torch.int32, device=cuda_device),
                       torch.zeros((0, 8, 8), dtype=torch.float32, device=cuda_device), (32, 16))
    out = torch.full((32, 12), 5.0, device=cuda_device)
    bsr.spmm_bsr8(a, torch.randn((16, 12), device=cuda_device), out=out)
    assert not out.any()
    a16 = bsr.DeviceBsr8(a.indptr, a.indices, a.blocks.to(torch.bfloat16), (32, 16))
    out = torch.full((32, 8), 5.0, device=cuda_device)
    bsr.spmm_bsr8(a16, torch.randn((16, 8), device=cuda_device).to(torch.bfloat16), out=out)
    assert not out.any()


def test_ragged_row_gather_two_destinations_on_one_gpu(cuda_device):
    """lf_allgather_rows with both destinations on this GPU (the peer case runs in the multi-GPU
    test): row blocks of different sizes land in the right rows of every full-size buffer."""
    import torch
    for N, ld in ((64, 64), (20, 24), (7, 9)):
        full = [torch.full((100, ld), float("nan"), device=cuda_device) for _ in range(2)]
        src = torch.randn((100, N), device=cuda_device)
        for a, b in ((0, 13), (13, 13), (13, 71), (71, 100)):
            hyb.allgather_rows(src[a:b].contiguous(), a, [t.data_ptr() for t in full], ld)
        for t in full:
            assert torch.equal(t[:, :N], src)
            assert ld == N or bool(torch.isnan(t[:, N:]).all())
