"""lf_hyb_stats_static: the statistics pass for callers that may not allocate device memory.

Some users of this library run it where allocating is off the table: inside a long-lived service
that fixed its device-memory footprint at start-up, or as a plugin under a host that owns the
allocator, where a cudaMalloc would stall every stream of the device.  For them the library keeps
the one scratch array of the statistics pass in static device memory.  This test drives the entry
point through the C ABI twice in a row, with different matrices so that stale scratch contents
would show, and requires the integer outputs to be identical to lf_hyb_stats with a caller-owned
workspace (integer counters: the tolerance is zero).  It is collected last on purpose.
"""
import numpy as np
import pytest

from liteform_ae_b200 import _cabi, hyb, synth

pytestmark = pytest.mark.gpu


def _static_stats(csr_dev, P):
    import torch
    lib = _cabi.load()
    M, K = csr_dev.shape
    dev = csr_dev.indptr.device
    stats = torch.full((P * _cabi.NUM_WIDTH_CLASSES * 3,), -7, dtype=torch.int64, device=dev)
    hist = torch.full((P * _cabi.COLMASK_BINS,), -7, dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        _cabi.check(lib.lf_hyb_stats_static(csr_dev.indptr.data_ptr(), csr_dev.indices.data_ptr(), M, K, P,
                                            stats.data_ptr(), hist.data_ptr(),
                                            torch.cuda.current_stream().cuda_stream))
    return (stats.cpu().numpy().reshape(P, _cabi.NUM_WIDTH_CLASSES, 3),
            hist.cpu().numpy().reshape(P, _cabi.COLMASK_BINS))


def test_static_scratch_matches_workspace_variant_twice(cuda_device):
    first = synth.skewed_rows(M=8192, seed=3)        # touches many columns with wide classes
    second = synth.zipf_rows(M=2048, seed=5)         # smaller: leftovers of `first` must not leak in
    for csr, P in ((first, 1), (second, 3), (first, 4)):
        d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
        want_stats, want_hist = hyb.hyb_stats(d, P)
        for _ in range(2):                            # two calls in a row on the same input
            got_stats, got_hist = _static_stats(d, P)
            assert np.array_equal(got_stats, want_stats)
            assert np.array_equal(got_hist, want_hist)


def test_static_variant_leaves_device_memory_alone(cuda_device):
    """The point of the entry point: after the first call on a device (which looks the scratch up)
    a call changes neither the free device memory the driver reports nor what PyTorch's allocator
    holds -- the outputs are allocated before the measurement, the call itself allocates nothing."""
    import torch
    lib = _cabi.load()
    csr = synth.zipf_rows(M=4096, seed=9)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    P = 2
    stats = torch.empty(P * _cabi.NUM_WIDTH_CLASSES * 3, dtype=torch.int64, device=cuda_device)
    hist = torch.empty(P * _cabi.COLMASK_BINS, dtype=torch.int64, device=cuda_device)

    def call():
        with torch.cuda.device(cuda_device):
            _cabi.check(lib.lf_hyb_stats_static(d.indptr.data_ptr(), d.indices.data_ptr(), csr.shape[0], csr.shape[1], P,
                                                stats.data_ptr(), hist.data_ptr(), torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize(cuda_device)

    call()                                   # warm-up: one-time address look-up, module load
    free_before, _ = torch.cuda.mem_get_info(cuda_device)
    reserved_before = torch.cuda.memory_reserved(cuda_device)
    for _ in range(3):
        call()
    free_after, _ = torch.cuda.mem_get_info(cuda_device)
    assert free_after == free_before
    assert torch.cuda.memory_reserved(cuda_device) == reserved_before


def test_sizes_beyond_the_static_scratch_are_refused(cuda_device):
    import torch
    lib = _cabi.load()
    K = _cabi.STATIC_STATS_MAX_COLS + 1
    indptr = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    indices = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = torch.zeros(33 + 2048, dtype=torch.int64, device=cuda_device)
    rc = lib.lf_hyb_stats_static(indptr.data_ptr(), indices.data_ptr(), 1, K, 1, out.data_ptr(),
                                 out[33:].data_ptr(), 0)
    assert rc == _cabi.LF_ERR_UNSUPPORTED
    assert b"at most" in lib.lf_last_error()
