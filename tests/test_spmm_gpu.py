"""SpMM through the C ABI vs SciPy (the reference's own golden product, MTX.dot).

Tolerance for float32: rel 1e-5 / abs 1e-4 (the benchmark contract); the comparison value is
SciPy's product evaluated in float64."""
import numpy as np
import pytest

from oracle import hyb_oracle as ho
from liteform_ae_b200 import hyb, synth
from tests import cases

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-5, 1e-4


def _coo(csr):
    return np.repeat(np.arange(csr.shape[0], dtype=np.int64), np.diff(csr.indptr)), csr.indices.astype(np.int64)


def _ref(csr, B):
    return ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, B.astype(np.float64))


def _setup(name, P, N, device, seed=0):
    import torch
    csr = cases.matrix(name)
    row, col = _coo(csr)
    widths = ho.search_bucket_config(row, col, csr.shape, P, max(N, 32))
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, device)
    fmt = hyb.build_hyb_device(d, widths, with_mask=False)
    B = synth.dense_features(csr.shape[1], N, seed)
    return csr, d, fmt, B, torch.from_numpy(B).to(device)


@pytest.mark.parametrize("name", cases.SMALL)
@pytest.mark.parametrize("N", [32, 64, 128, 256, 512])
def test_hyb_spmm_matches_scipy(cuda_device, name, N):
    for P in (1, 4):
        csr, d, fmt, B, Bd = _setup(name, P, N, cuda_device)
        C = hyb.spmm_hyb(fmt, Bd)
        np.testing.assert_allclose(C.cpu().numpy(), _ref(csr, B), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("N", [1, 3, 20, 33, 96, 100, 130, 640, 1024])
def test_odd_feature_widths(cuda_device, N):
    csr, d, fmt, B, Bd = _setup("zipf_2048_s5", 1, N, cuda_device)
    C = hyb.spmm_hyb(fmt, Bd)
    np.testing.assert_allclose(C.cpu().numpy(), _ref(csr, B), rtol=RTOL, atol=ATOL)
    C2 = hyb.spmm_csr(d, Bd)
    np.testing.assert_allclose(C2.cpu().numpy(), _ref(csr, B), rtol=RTOL, atol=ATOL)


def test_output_is_overwritten_not_accumulated(cuda_device):
    import torch
    csr, d, fmt, B, Bd = _setup("skew_8192_s3", 1, 64, cuda_device)
    C = torch.full((csr.shape[0], 64), 7.0, device=cuda_device)
    for _ in range(3):
        hyb.spmm_hyb(fmt, Bd, out=C)
    np.testing.assert_allclose(C.cpu().numpy(), _ref(csr, B), rtol=RTOL, atol=ATOL)


def test_accumulate_flag_adds(cuda_device):
    import torch
    for P in (1, 2):
        csr, d, fmt, B, Bd = _setup("powerlaw_8192_s1", P, 128, cuda_device)
        C = torch.ones((csr.shape[0], 128), device=cuda_device)
        hyb.spmm_hyb(fmt, Bd, out=C, accumulate=True)
        np.testing.assert_allclose(C.cpu().numpy(), _ref(csr, B) + 1.0, rtol=RTOL, atol=ATOL)


def test_strided_operands(cuda_device):
    import torch
    csr, d, fmt, B, Bd = _setup("zipf_2048_s5", 1, 64, cuda_device)
    Bbig = torch.zeros((csr.shape[1], 96), device=cuda_device)
    Bbig[:, 8:72] = Bd                       # ldb = 96, 32-byte offset
    Cbig = torch.full((csr.shape[0], 80), -1.0, device=cuda_device)
    hyb.spmm_hyb(fmt, Bbig[:, 8:72], out=Cbig[:, 4:68])
    got = Cbig.cpu().numpy()
    np.testing.assert_allclose(got[:, 4:68], _ref(csr, B), rtol=RTOL, atol=ATOL)
    assert (got[:, :4] == -1).all() and (got[:, 68:] == -1).all()
    # odd leading dimension forces the scalar kernel
    Bodd = torch.zeros((csr.shape[1], 65), device=cuda_device)
    Bodd[:, :64] = Bd
    C = hyb.spmm_hyb(fmt, Bodd[:, :64])
    np.testing.assert_allclose(C.cpu().numpy(), _ref(csr, B), rtol=RTOL, atol=ATOL)


def test_explicit_zero_values_and_empty_rows(cuda_device):
    """A stored 0.0 must not leave its row unwritten; rows without entries must come out 0."""
    import torch
    csr = synth.zipf_rows(M=1024, seed=9)
    data = csr.data.copy()
    data[::3] = 0.0
    lens = np.diff(csr.indptr)
    lone = np.nonzero(lens == 1)[0]
    data[csr.indptr[lone]] = 0.0             # rows whose only entry is an explicit zero
    keep = np.ones(csr.nnz, dtype=bool)
    for r in (5, 6, 700):                    # carve empty rows
        keep[csr.indptr[r]:csr.indptr[r + 1]] = False
    rows = np.repeat(np.arange(1024), lens)[keep]
    indptr = np.zeros(1025, dtype=np.int64)
    np.cumsum(np.bincount(rows, minlength=1024), out=indptr[1:])
    csr2 = synth.Csr(indptr, csr.indices[keep], data[keep], csr.shape)
    row, col = _coo(csr2)
    widths = ho.search_bucket_config(row, col, csr2.shape, 1, 32)
    d = hyb.DeviceCsr.from_host(csr2.indptr, csr2.indices, csr2.data, csr2.shape, cuda_device)
    fmt = hyb.build_hyb_device(d, widths)
    B = synth.dense_features(1024, 32, 3)
    C = torch.full((1024, 32), float("nan"), device=cuda_device)
    hyb.spmm_hyb(fmt, torch.from_numpy(B).to(cuda_device), out=C)
    got = C.cpu().numpy()
    assert not np.isnan(got).any()
    np.testing.assert_allclose(got, _ref(csr2, B), rtol=RTOL, atol=ATOL)
    assert not got[[5, 6, 700]].any()


def test_long_rows_split_over_many_groups(cuda_device):
    """Rows far longer than the widest bucket: runs of equal row ids cut by group boundaries."""
    import torch
    csr = synth.skewed_rows(M=4096, seed=5, heavy_rows=6, heavy_len=3000)
    row, col = _coo(csr)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    B = synth.dense_features(4096, 128, 4)
    Bd = torch.from_numpy(B).to(cuda_device)
    for widths in ([[1, 2, 4, 8, 16]], [[4]], [[1]], [[1024]], [[2, 512]]):
        fmt = hyb.build_hyb_device(d, widths)
        C = hyb.spmm_hyb(fmt, Bd)
        np.testing.assert_allclose(C.cpu().numpy(), _ref(csr, B), rtol=RTOL, atol=ATOL)


def test_row_shards(cuda_device):
    import torch
    csr, d, fmt, B, Bd = _setup("skew_8192_s3", 1, 64, cuda_device)
    cuts = hyb.shard_rows(d, 4)
    out = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        part = hyb.build_hyb_device(d, fmt.bucket_widths, row_range=(a, b), with_mask=False)
        out.append(hyb.spmm_hyb(part, Bd).cpu().numpy())
    np.testing.assert_allclose(np.concatenate(out), _ref(csr, B), rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("N,pinned", [(32, False), (64, True), (100, True)])
def test_host_memory_entry_point(cuda_device, N, pinned):
    import torch
    csr, d, fmt, B, Bd = _setup("zipf_16384_s0", 1, N, cuda_device)
    r, c, m, v = fmt.to_nested_numpy(with_values=True)
    ell_rows, row_off, slot_off, rows, cols, vals, zero_rows = hyb.HybFormat.host_layout(
        fmt.bucket_widths, r, c, v, csr.shape[0])
    host_fmt = hyb.HybFormat(csr.shape, (0, csr.shape[0]), fmt.bucket_widths, ell_rows, row_off, slot_off,
                             None, None, None, None, zero_rows)
    ws = torch.empty(hyb.host_workspace_bytes(host_fmt, N), dtype=torch.uint8, device=cuda_device)
    if pinned:
        Bh = torch.from_numpy(B).pin_memory().numpy()
        Ch = torch.full((csr.shape[0], N), float("nan")).pin_memory().numpy()
    else:
        Bh, Ch = B, np.full((csr.shape[0], N), np.nan, dtype=np.float32)
    for _ in range(2):
        hyb.spmm_hyb_host((rows, cols, vals, zero_rows), host_fmt, Bh, Ch, ws)
        np.testing.assert_allclose(Ch, _ref(csr, B), rtol=RTOL, atol=ATOL)
        Ch[:] = np.nan


def test_host_memory_entry_point_two_calls_in_flight(cuda_device):
    """LF_SPMM_NO_SYNC: two products enqueued on two streams with their own workspaces and result
    buffers, then one synchronisation; both results must be complete and correct."""
    import torch
    N = 64
    csr, d, fmt, B, Bd = _setup("zipf_16384_s0", 1, N, cuda_device)
    r, c, m, v = fmt.to_nested_numpy(with_values=True)
    ell_rows, row_off, slot_off, rows, cols, vals, zero_rows = hyb.HybFormat.host_layout(
        fmt.bucket_widths, r, c, v, csr.shape[0])
    host_fmt = hyb.HybFormat(csr.shape, (0, csr.shape[0]), fmt.bucket_widths, ell_rows, row_off, slot_off,
                             None, None, None, None, zero_rows)
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory().numpy()
    h = tuple(pin(a) for a in (rows, cols, vals, zero_rows))
    Bs = [pin(B), pin(2.0 * B)]
    Cs = [pin(np.full((csr.shape[0], N), np.nan, dtype=np.float32)) for _ in range(2)]
    ws = [torch.empty(hyb.host_workspace_bytes(host_fmt, N), dtype=torch.uint8, device=cuda_device) for _ in range(2)]
    streams = [torch.cuda.Stream(device=cuda_device) for _ in range(2)]
    for rep in range(3):
        for k in (0, 1):
            hyb.spmm_hyb_host(h, host_fmt, Bs[k], Cs[k], ws[k], sync=False, stream=streams[k])
    for st in streams:
        st.synchronize()
    want = _ref(csr, B)
    np.testing.assert_allclose(Cs[0], want, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(Cs[1], 2.0 * want, rtol=RTOL, atol=2 * ATOL)
    lib = __import__("liteform_ae_b200._cabi", fromlist=["load"]).load()
    s = host_fmt.c_struct(host_arrays=h)
    import ctypes
    assert lib.lf_spmm_hyb_f32_host(ctypes.byref(s), Bs[0].ctypes.data, Cs[0].ctypes.data, N, 8,
                                    ws[0].data_ptr(), ws[0].numel(), None) == -1     # unknown flag bits


def test_full_size_linearity_and_checksum(cuda_device):
    """Benchmark-size power-law matrix: properties that need no CPU product of the same size.
    (1) column sums: 1^T (A B) == (1^T A) B in float64; (2) linearity in B; (3) sampled rows."""
    import torch
    csr = cases.matrix("powerlaw_1048576_s1")
    N = 128
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    from liteform_ae_b200 import width_search as ws
    stats, hist = hyb.hyb_stats(d, 1)
    fmt = hyb.build_hyb_device(d, ws.search_from_stats(stats, hist, N, 1), with_mask=False)
    B = synth.dense_features(csr.shape[1], N, 7)
    Bd = torch.from_numpy(B).to(cuda_device)
    C = hyb.spmm_hyb(fmt, Bd)
    colsum_A = np.bincount(csr.indices, weights=csr.data.astype(np.float64), minlength=csr.shape[1])
    want = colsum_A @ B.astype(np.float64)
    got = C.double().sum(dim=0).cpu().numpy()
    np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-3)
    C2 = hyb.spmm_hyb(fmt, 2.0 * Bd)
    # scaling B by 2 is exact in floating point; rows owned by one ELL row are summed in a fixed
    # order and must scale bit for bit, rows assembled with atomics may differ in the last bits
    owned = torch.ones(csr.shape[0], dtype=torch.bool, device=cuda_device)
    owned[fmt.zero_rows.long()] = False
    assert torch.equal(C2[owned], 2.0 * C[owned])
    torch.testing.assert_close(C2[~owned], 2.0 * C[~owned], rtol=1e-5, atol=1e-6)
    rng = np.random.default_rng(0)
    pick = np.unique(np.concatenate([rng.integers(0, csr.shape[0], 2000), np.argsort(np.diff(csr.indptr))[-8:]]))
    sub = synth.Csr(np.concatenate([[0], np.cumsum(np.diff(csr.indptr)[pick])]),
                    np.concatenate([csr.indices[csr.indptr[r]:csr.indptr[r + 1]] for r in pick]),
                    np.concatenate([csr.data[csr.indptr[r]:csr.indptr[r + 1]] for r in pick]),
                    (len(pick), csr.shape[1]))
    np.testing.assert_allclose(C[torch.from_numpy(pick).to(cuda_device)].cpu().numpy(), _ref(sub, B),
                               rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("N", [64, 128, 200])
def test_broadcasting_spmm_two_destinations_on_one_gpu(cuda_device, N):
    """lf_spmm_hyb_f32_bcast with both destinations on this GPU (the peer case needs two GPUs and is
    exercised by bench.py --gather fused): every shard writes its rows into both full-size buffers.
    64 features run the register kernel, 128 and 200 the shared-memory-ring kernel."""
    import torch
    for P, name in ((1, "skew_8192_s3"), (2, "powerlaw_8192_s1")):
        csr, d, fmt, B, Bd = _setup(name, P, N, cuda_device)
        full = [torch.full((csr.shape[0], N), float("nan"), device=cuda_device) for _ in range(2)]
        cuts = hyb.shard_rows(d, 3)
        for a, b in zip(cuts[:-1], cuts[1:]):
            part = hyb.build_hyb_device(d, fmt.bucket_widths, row_range=(a, b), with_mask=False)
            hyb.spmm_hyb_bcast(part, Bd, [t.data_ptr() for t in full], N)
        want = _ref(csr, B)
        for t in full:
            np.testing.assert_allclose(t.cpu().numpy(), want, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("N", [8, 64, 128, 256, 512, 1000])
def test_bf16_features_fp32_accumulate(cuda_device, N):
    """B in bf16, values and accumulation in float32: rel 1e-2 against the float64 product of the
    unrounded B, and 1e-5 against the product of the rounded B (isolates the accumulation)."""
    import torch
    for name, P in (("skew_8192_s3", 1), ("powerlaw_8192_s1", 3)):
        csr, d, fmt, B, Bd = _setup(name, P, N, cuda_device)
        B16 = Bd.to(torch.bfloat16)
        C = hyb.spmm_hyb(fmt, B16).cpu().numpy()
        want = _ref(csr, B)
        assert np.abs(C - want).max() <= 1e-2 * np.abs(want).max()
        rounded = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape,
                                    B16.float().cpu().numpy().astype(np.float64))
        np.testing.assert_allclose(C, rounded, rtol=RTOL, atol=ATOL)
    with pytest.raises(Exception, match="multiples of 8"):
        hyb.spmm_hyb(fmt, torch.zeros((csr.shape[1], 12), dtype=torch.bfloat16, device=cuda_device))


@pytest.mark.parametrize("N", [32, 64, 128, 200, 512])
def test_csr_spmm_balanced_over_entries(cuda_device, N):
    """Long rows shared by many groups, empty rows (leading, trailing, in between), row ranges."""
    import torch
    csr = synth.skewed_rows(M=4096, seed=11, heavy_rows=5, heavy_len=3000)
    lens = np.diff(csr.indptr).copy()
    for r in (0, 1, 2, 77, 78, 4094, 4095):       # carve empty rows
        lens[r] = 0
    keep = np.repeat(lens > 0, np.diff(csr.indptr))
    indptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int64)
    csr2 = synth.Csr(indptr, csr.indices[keep], csr.data[keep], csr.shape)
    d = hyb.DeviceCsr.from_host(csr2.indptr, csr2.indices, csr2.data, csr2.shape, cuda_device)
    B = synth.dense_features(4096, N, 5)
    Bd = torch.from_numpy(B).to(cuda_device)
    want = _ref(csr2, B)
    C = torch.full((4096, N), float("nan"), device=cuda_device)
    hyb.spmm_csr(d, Bd, out=C)
    np.testing.assert_allclose(C.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    part = hyb.spmm_csr(d, Bd, row_range=(70, 3000)).cpu().numpy()
    np.testing.assert_allclose(part, want[70:3000], rtol=RTOL, atol=ATOL)
    ones = hyb.DeviceCsr(d.indptr, d.indices, None, d.shape)      # data = NULL: all ones
    pattern = synth.Csr(csr2.indptr, csr2.indices, np.ones(csr2.nnz, dtype=np.float32), csr2.shape)
    np.testing.assert_allclose(hyb.spmm_csr(ones, Bd).cpu().numpy(), _ref(pattern, B), rtol=RTOL, atol=ATOL)
