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
