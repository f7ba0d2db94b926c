"""Device-resident composed format and the calls that build and multiply it.

PyTorch is used here for device memory and streams only; every computation is a call
into ``liblf_b200.so``.  The functions raise if CUDA or the library is unavailable.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np

from . import _cabi
from ._cabi import LfHyb, check, np_ptr, t_ptr

BUCKET_ALIGN = 64


def _torch():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("liteform_ae_b200 needs a CUDA device (there is no CPU path)")
    return torch


def _stream_ptr(torch) -> int:
    return torch.cuda.current_stream().cuda_stream


@dataclass
class DeviceCsr:
    """CSR matrix in device memory: int64 row pointers, int32 sorted distinct columns."""
    indptr: "object"            # torch int64 [M + 1]
    indices: "object"           # torch int32 [nnz]
    data: Optional["object"]    # torch float32 [nnz] or None (all ones)
    shape: Tuple[int, int]

    @property
    def nnz(self) -> int:
        return int(self.indices.numel())

    @staticmethod
    def from_host(indptr, indices, data, shape, device="cuda", validate: bool = True) -> "DeviceCsr":
        """Upload host arrays.  Column indices that do not fit int32 are refused here (a cast would
        wrap them); with ``validate`` the uploaded matrix is checked on the device by
        ``lf_csr_validate`` (row pointers, column range, strictly ascending columns)."""
        torch = _torch()
        indices = np.asarray(indices)
        if indices.dtype != np.int32 and indices.size and (int(indices.max()) > 0x7fffffff or int(indices.min()) < 0):
            raise ValueError("column indices must lie in [0, 2^31)")
        ip = torch.from_numpy(np.ascontiguousarray(indptr, dtype=np.int64)).to(device)
        ix = torch.from_numpy(np.ascontiguousarray(indices, dtype=np.int32)).to(device)
        dv = None if data is None else torch.from_numpy(np.ascontiguousarray(data, dtype=np.float32)).to(device)
        csr = DeviceCsr(ip, ix, dv, (int(shape[0]), int(shape[1])))
        if validate:
            csr.validate()
        return csr

    def validate(self) -> None:
        """``lf_csr_validate``: raises ``ValueError`` when the matrix is not canonical CSR."""
        torch = _torch()
        lib = _cabi.load()
        assert self.indptr.numel() == self.shape[0] + 1, "indptr must hold one entry per row plus one"
        with torch.cuda.device(self.indptr.device):
            st = lib.lf_csr_validate(t_ptr(self.indptr), t_ptr(self.indices), self.shape[0], self.shape[1],
                                     self.nnz, _stream_ptr(torch))
        if st == _cabi.LF_ERR_INVALID_ARGUMENT:
            raise ValueError(lib.lf_last_error().decode("utf-8", "replace"))
        check(st)


def flatten_widths(bucket_widths: Sequence[Sequence[int]]):
    pbo = np.zeros(len(bucket_widths) + 1, dtype=np.int32)
    np.cumsum([len(w) for w in bucket_widths], out=pbo[1:])
    flat = np.asarray([w for ws in bucket_widths for w in ws], dtype=np.int32)
    return pbo, flat


class Workspace:
    """A device byte buffer that grows on demand and is handed to consecutive builder calls, so that
    a sequence of builds (statistics, plan, fill) on one stream allocates once instead of per call.
    Not for concurrent use from several streams."""

    def __init__(self, device):
        self.device = device
        self._buf = None
        self._cursor = 0

    def get(self, nbytes: int, slot: int = 0):
        """A 256-byte aligned view of ``nbytes`` bytes.  ``slot == 0`` starts over at the beginning
        of the buffer; views requested with increasing slot numbers after it do not overlap.  A view
        stays valid when a later request makes the buffer grow (it keeps the old storage alive)."""
        torch = _torch()
        if slot == 0:
            self._cursor = 0
        start = -(-self._cursor // 256) * 256
        end = start + max(int(nbytes), 1)
        if self._buf is None or self._buf.numel() < end:
            have = 0 if self._buf is None else self._buf.numel()
            self._buf = torch.empty(max(end, 2 * have), dtype=torch.uint8, device=self.device)
        self._cursor = end
        return self._buf[start:end]


def hyb_stats(csr: DeviceCsr, num_parts: int, workspace: Optional[Workspace] = None):
    """Run ``lf_hyb_stats``; returns ``(class_stats int64[P,11,3], colmask_hist int64[P,2048])`` on the host."""
    torch = _torch()
    lib = _cabi.load()
    M, K = csr.shape
    dev = csr.indptr.device
    n_stat, n_hist = num_parts * _cabi.NUM_WIDTH_CLASSES * 3, num_parts * _cabi.COLMASK_BINS
    with torch.cuda.device(dev):
        ws_bytes = lib.lf_hyb_stats_workspace_bytes(M, K, num_parts)
        if workspace is None:
            out = torch.empty(n_stat + n_hist, dtype=torch.int64, device=dev)
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        else:
            out = workspace.get((n_stat + n_hist) * 8, 0).view(torch.int64)
            ws = workspace.get(ws_bytes, 1)
        check(lib.lf_hyb_stats(t_ptr(csr.indptr), t_ptr(csr.indices), M, K, num_parts, out.data_ptr(),
                               out.data_ptr() + n_stat * 8, ws.data_ptr(), ws_bytes, _stream_ptr(torch)))
        host = out.cpu().numpy()      # one read-back for both tables (synchronises the stream)
        return (host[:n_stat].reshape(num_parts, _cabi.NUM_WIDTH_CLASSES, 3).copy(),
                host[n_stat:].reshape(num_parts, _cabi.COLMASK_BINS).copy())


class HybFormat:
    """A composed-format matrix (or a row shard of one) in device memory.

    Layout: buckets are numbered partition-major (``part_bucket_off``); bucket ``i`` owns
    ``rows[row_off[i] : row_off[i] + ell_rows[i]]`` and the ``[ell_rows[i], widths[i]]`` tiles of
    ``cols`` / ``vals`` / ``mask`` starting at ``slot_off[i]``.
    """

    def __init__(self, shape, row_range, bucket_widths, ell_rows, row_off, slot_off, rows, cols, vals,
                 mask, zero_rows):
        self.shape = (int(shape[0]), int(shape[1]))
        self.row_begin, self.row_end = int(row_range[0]), int(row_range[1])
        self.bucket_widths = [list(map(int, w)) for w in bucket_widths]
        self.num_parts = len(self.bucket_widths)
        self.part_bucket_off, self.widths = flatten_widths(self.bucket_widths)
        self.ell_rows = np.ascontiguousarray(ell_rows, dtype=np.int64)
        self.row_off = np.ascontiguousarray(row_off, dtype=np.int64)
        self.slot_off = np.ascontiguousarray(slot_off, dtype=np.int64)
        self.rows, self.cols, self.vals, self.mask, self.zero_rows = rows, cols, vals, mask, zero_rows

    # -- C view ---------------------------------------------------------------------------
    def c_struct(self, host_arrays=None) -> LfHyb:
        """``struct lf_hyb`` over this object's buffers (keep ``self`` alive while it is used).
        ``host_arrays=(rows, cols, vals, zero_rows)`` substitutes NumPy buffers for the
        device ones (for the host-memory entry point)."""
        s = LfHyb()
        s.num_rows, s.num_cols = self.shape
        s.row_begin, s.row_end = self.row_begin, self.row_end
        s.num_parts = self.num_parts
        s.num_buckets = int(len(self.widths))
        s.part_bucket_off = np_ptr(self.part_bucket_off)
        s.widths = np_ptr(self.widths)
        s.ell_rows = np_ptr(self.ell_rows)
        s.row_off = np_ptr(self.row_off)
        s.slot_off = np_ptr(self.slot_off)
        if host_arrays is None:
            s.rows, s.cols, s.vals = t_ptr(self.rows), t_ptr(self.cols), t_ptr(self.vals)
            s.mask = t_ptr(self.mask)
            s.zero_rows = t_ptr(self.zero_rows) if self.num_zero_rows else 0
        else:
            r, c, v, z = host_arrays
            s.rows, s.cols, s.vals, s.mask = np_ptr(r), np_ptr(c), np_ptr(v), 0
            s.zero_rows = np_ptr(z) if self.num_zero_rows else 0
        s.num_zero_rows = self.num_zero_rows
        return s

    @property
    def num_zero_rows(self) -> int:
        return 0 if self.zero_rows is None else int(self.zero_rows.shape[0])

    @property
    def total_slots(self) -> int:
        return int((self.ell_rows * self.widths).sum())

    @property
    def device(self):
        return self.cols.device

    # -- host views -----------------------------------------------------------------------
    def to_nested_numpy(self, with_values: bool = False):
        """``(row_indices_nd, col_indices_nd, mask_nd[, values_nd])`` nested ``[partition][bucket]``
        exactly as ``build_hyb_format`` returns them (format_algos.py:385), as int32 arrays."""
        rows = self.rows.cpu().numpy()
        cols = self.cols.cpu().numpy()
        mask = None if self.mask is None else self.mask.cpu().numpy()
        vals = self.vals.cpu().numpy()
        R, Cc, Mk, V = [], [], [], []
        for p in range(self.num_parts):
            rp, cp, mp, vp_ = [], [], [], []
            for i in range(self.part_bucket_off[p], self.part_bucket_off[p + 1]):
                n, w = int(self.ell_rows[i]), int(self.widths[i])
                ro, so = int(self.row_off[i]), int(self.slot_off[i])
                rp.append(rows[ro:ro + n].copy())
                cp.append(cols[so:so + n * w].reshape(n, w).copy())
                if mask is not None:
                    mp.append(mask[so:so + n * w].reshape(n, w).astype(np.int32))
                vp_.append(vals[so:so + n * w].reshape(n, w).copy())
            R.append(rp); Cc.append(cp); Mk.append(mp); V.append(vp_)
        return (R, Cc, Mk, V) if with_values else (R, Cc, Mk)

    @staticmethod
    def host_layout(bucket_widths, rows_nd, cols_nd, vals_nd, num_rows: int, row_range=None):
        """Pack nested host arrays into the flat arenas (bucket starts aligned to 64 elements).

        Returns ``(ell_rows, row_off, slot_off, rows, cols, vals, zero_rows)`` as NumPy arrays.
        ``zero_rows`` are the rows of the range that do not have exactly one ELL row.
        """
        pbo, flat_w = flatten_widths(bucket_widths)
        nb = len(flat_w)
        ell_rows = np.zeros(nb, dtype=np.int64)
        row_off = np.zeros(nb + 1, dtype=np.int64)
        slot_off = np.zeros(nb + 1, dtype=np.int64)
        i = 0
        for p, ws in enumerate(bucket_widths):
            for b, w in enumerate(ws):
                n = int(np.asarray(rows_nd[p][b]).shape[0])
                ell_rows[i] = n
                row_off[i + 1] = row_off[i] + -(-n // BUCKET_ALIGN) * BUCKET_ALIGN
                slot_off[i + 1] = slot_off[i] + -(-(n * w) // BUCKET_ALIGN) * BUCKET_ALIGN
                i += 1
        rows = np.zeros(int(row_off[-1]), dtype=np.int32)
        cols = np.zeros(int(slot_off[-1]), dtype=np.int32)
        vals = np.zeros(int(slot_off[-1]), dtype=np.float32)
        i = 0
        for p, ws in enumerate(bucket_widths):
            for b, w in enumerate(ws):
                n = int(ell_rows[i])
                rows[row_off[i]:row_off[i] + n] = np.asarray(rows_nd[p][b]).astype(np.int32)
                cols[slot_off[i]:slot_off[i] + n * w] = np.asarray(cols_nd[p][b]).astype(np.int32).reshape(-1)
                vals[slot_off[i]:slot_off[i] + n * w] = np.asarray(vals_nd[p][b]).astype(np.float32).reshape(-1)
                i += 1
        r0, r1 = (0, num_rows) if row_range is None else row_range
        count = np.zeros(r1 - r0, dtype=np.int64)
        for i in range(nb):
            n = int(ell_rows[i])
            if n:
                count += np.bincount(rows[row_off[i]:row_off[i] + n].astype(np.int64) - r0, minlength=r1 - r0)
        zero_rows = (np.nonzero(count != 1)[0] + r0).astype(np.int32)
        return ell_rows, row_off, slot_off, rows, cols, vals, zero_rows

    @staticmethod
    def from_nested_numpy(bucket_widths, rows_nd, cols_nd, mask_or_vals_nd, shape, device="cuda",
                          row_range=None) -> "HybFormat":
        """Upload a format that lives in host memory (what ``bench_hyb_with_config`` receives)."""
        torch = _torch()
        ell_rows, row_off, slot_off, rows, cols, vals, zero_rows = HybFormat.host_layout(
            bucket_widths, rows_nd, cols_nd, mask_or_vals_nd, shape[0], row_range)
        up = lambda a: torch.from_numpy(a).to(device)
        rr = (0, shape[0]) if row_range is None else row_range
        return HybFormat(shape, rr, bucket_widths, ell_rows, row_off, slot_off, up(rows), up(cols),
                         up(vals), None, up(zero_rows))


def build_hyb_device(csr: DeviceCsr, bucket_widths: Sequence[Sequence[int]],
                     row_range: Optional[Tuple[int, int]] = None, with_mask: bool = True,
                     workspace: Optional[Workspace] = None) -> HybFormat:
    """``lf_hyb_plan`` + ``lf_hyb_fill``: CSR in device memory -> composed format in device memory.
    With a ``Workspace`` the scratch of both calls comes out of it and the call returns without
    waiting for the fill (stream order protects the scratch for the next call on the same stream)."""
    torch = _torch()
    lib = _cabi.load()
    M, K = csr.shape
    r0, r1 = (0, M) if row_range is None else (int(row_range[0]), int(row_range[1]))
    P = len(bucket_widths)
    pbo, flat_w = flatten_widths(bucket_widths)
    nb = int(len(flat_w))
    dev = csr.indptr.device
    with torch.cuda.device(dev):
        stream = _stream_ptr(torch)
        ws_bytes = lib.lf_hyb_build_workspace_bytes(r0, r1, P, nb)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if workspace is None else workspace.get(ws_bytes, 0)
        ell_rows = np.zeros(max(nb, 1), dtype=np.int64)
        row_off = np.zeros(nb + 1, dtype=np.int64)
        slot_off = np.zeros(nb + 1, dtype=np.int64)
        n_zero = C.c_int64(0)
        check(lib.lf_hyb_plan(t_ptr(csr.indptr), t_ptr(csr.indices), M, K, r0, r1, P, np_ptr(pbo),
                              np_ptr(flat_w) if nb else 0, np_ptr(ell_rows), np_ptr(row_off),
                              np_ptr(slot_off), C.addressof(n_zero), ws.data_ptr(), ws_bytes, stream))
        ell_rows = ell_rows[:nb]
        n_rows_total, n_slots_total = int(row_off[nb]), int(slot_off[nb])
        rows = torch.empty(n_rows_total, dtype=torch.int32, device=dev)
        cols = torch.empty(n_slots_total, dtype=torch.int32, device=dev)
        vals = torch.empty(n_slots_total, dtype=torch.float32, device=dev)
        mask = torch.empty(n_slots_total, dtype=torch.uint8, device=dev) if with_mask else None
        zero_rows = torch.empty(int(n_zero.value), dtype=torch.int32, device=dev)
        fmt = HybFormat((M, K), (r0, r1), bucket_widths, ell_rows, row_off, slot_off, rows, cols, vals,
                        mask, zero_rows)
        sc_bytes = lib.lf_hyb_fill_scratch_bytes(n_rows_total)
        scratch = torch.empty(sc_bytes, dtype=torch.uint8, device=dev) if workspace is None else workspace.get(sc_bytes, 1)
        layout = fmt.c_struct()
        check(lib.lf_hyb_fill(t_ptr(csr.indptr), t_ptr(csr.indices), t_ptr(csr.data), C.byref(layout),
                              ws.data_ptr(), ws_bytes, scratch.data_ptr(), sc_bytes, stream))
        if workspace is None:
            torch.cuda.current_stream().synchronize()   # ws / scratch are released on return
    return fmt


def spmm_hyb(fmt: HybFormat, B, out=None, accumulate: bool = False):
    """``lf_spmm_hyb_f32`` (or ``lf_spmm_hyb_bf16`` when B is bfloat16): returns
    ``C[row_begin:row_end]`` (float32, on the format's device)."""
    torch = _torch()
    lib = _cabi.load()
    assert B.is_cuda and B.dtype in (torch.float32, torch.bfloat16) and B.dim() == 2 and B.stride(1) == 1
    assert B.shape[0] == fmt.shape[1], "B must have one row per matrix column"
    N = int(B.shape[1])
    n_rows = fmt.row_end - fmt.row_begin
    if out is None:
        if accumulate:
            raise ValueError("accumulate=True needs an output tensor")
        out = torch.empty((n_rows, N), dtype=torch.float32, device=B.device)
    assert out.shape == (n_rows, N) and out.stride(1) == 1 and out.dtype == torch.float32
    with torch.cuda.device(B.device):
        s = fmt.c_struct()
        fn = lib.lf_spmm_hyb_f32 if B.dtype == torch.float32 else lib.lf_spmm_hyb_bf16
        check(fn(C.byref(s), B.data_ptr(), B.stride(0), out.data_ptr(), out.stride(0), N,
                                  _cabi.LF_SPMM_ACCUMULATE if accumulate else _cabi.LF_SPMM_OVERWRITE,
                                  _stream_ptr(torch)))
    return out


def spmm_hyb_kernel_name(fmt: HybFormat, B, out) -> str:
    """``lf_spmm_hyb_f32_kernel_name``: the kernel ``spmm_hyb(fmt, B, out=out)`` launches for float32 B."""
    s = fmt.c_struct()
    name = _cabi.load().lf_spmm_hyb_f32_kernel_name(C.byref(s), B.data_ptr(), B.stride(0), out.data_ptr(),
                                                    out.stride(0), int(B.shape[1]))
    return name.decode()


def spmm_csr(csr: DeviceCsr, B, out=None, row_range=None):
    """``lf_spmm_csr_f32`` on rows ``row_range`` (default: all)."""
    torch = _torch()
    lib = _cabi.load()
    assert B.is_cuda and B.dtype == torch.float32 and B.stride(1) == 1
    r0, r1 = (0, csr.shape[0]) if row_range is None else row_range
    N = int(B.shape[1])
    if out is None:
        out = torch.empty((r1 - r0, N), dtype=torch.float32, device=B.device)
    with torch.cuda.device(B.device):
        nnz = csr.nnz if (r0, r1) == (0, csr.shape[0]) else -1
        check(lib.lf_spmm_csr_f32(t_ptr(csr.indptr), t_ptr(csr.indices), t_ptr(csr.data), r0, r1, nnz,
                                  B.data_ptr(), B.stride(0), out.data_ptr(), out.stride(0), N,
                                  _stream_ptr(torch)))
    return out


def spmm_hyb_host(fmt_host_arrays, fmt: HybFormat, B_host: np.ndarray, C_host: np.ndarray, workspace,
                  accumulate: bool = False, sync: bool = True, stream=None, format_resident: bool = False):
    """``lf_spmm_hyb_f32_host``: all operands in (ideally pinned) host memory; ``workspace`` is a
    device byte tensor of at least ``host_workspace_bytes(fmt, N)`` bytes.  ``sync=False`` only
    enqueues on ``stream`` (a ``torch.cuda.Stream``, default: the current one): ``C_host`` is valid
    and the workspace reusable after that stream has been synchronised.  ``format_resident=True``
    skips the upload of the format: ``workspace`` must still hold it from an earlier call with the
    same format and N."""
    torch = _torch()
    lib = _cabi.load()
    N = int(B_host.shape[1])
    s = fmt.c_struct(host_arrays=fmt_host_arrays)
    flags = (_cabi.LF_SPMM_ACCUMULATE if accumulate else _cabi.LF_SPMM_OVERWRITE) | (0 if sync else _cabi.LF_SPMM_NO_SYNC) \
        | (_cabi.LF_SPMM_FORMAT_RESIDENT if format_resident else 0)
    with torch.cuda.device(workspace.device):
        st = _stream_ptr(torch) if stream is None else stream.cuda_stream
        check(lib.lf_spmm_hyb_f32_host(C.byref(s), np_ptr(B_host), np_ptr(C_host), N, flags,
                                       workspace.data_ptr(), workspace.numel(), st))
    return C_host


def host_workspace_bytes(fmt: HybFormat, N: int) -> int:
    s = fmt.c_struct(host_arrays=(None, None, None, None))
    return int(_cabi.load().lf_spmm_hyb_f32_host_workspace_bytes(C.byref(s), N))


def shard_rows(csr: DeviceCsr, num_shards: int) -> List[int]:
    """``lf_shard_rows``: nnz-balanced contiguous row split points (``num_shards + 1`` values)."""
    torch = _torch()
    lib = _cabi.load()
    out = torch.empty(num_shards + 1, dtype=torch.int64, device=csr.indptr.device)
    with torch.cuda.device(out.device):
        check(lib.lf_shard_rows(t_ptr(csr.indptr), csr.shape[0], num_shards, t_ptr(out), _stream_ptr(torch)))
    return [int(x) for x in out.cpu().tolist()]


def row_length_stats(csr: DeviceCsr, row_range=None):
    """``lf_row_stats`` folded on the host: exact ``(count, sum, sum_of_squares, min, max)`` of the row
    lengths as Python integers."""
    torch = _torch()
    lib = _cabi.load()
    r0, r1 = (0, csr.shape[0]) if row_range is None else row_range
    nblk = int(lib.lf_row_stats_blocks(r0, r1))
    if nblk == 0:
        return 0, 0, 0, 0, 0
    part = torch.empty(nblk * 4, dtype=torch.int64, device=csr.indptr.device)
    with torch.cuda.device(part.device):
        check(lib.lf_row_stats(t_ptr(csr.indptr), r0, r1, t_ptr(part), _stream_ptr(torch)))
    p = part.cpu().numpy().view(np.uint64).reshape(nblk, 4)
    return (r1 - r0, sum(int(x) for x in p[:, 0]), sum(int(x) for x in p[:, 1]),
            int(p[:, 2].min()), int(p[:, 3].max()))


def spmm_hyb_bcast(fmt: HybFormat, B, dest_ptrs: Sequence[int], ldc: int):
    """``lf_spmm_hyb_f32_bcast``: write this shard's rows of C = A @ B into every full-size C whose
    device address is listed in ``dest_ptrs`` (own buffer and peers' symmetric-memory buffers)."""
    torch = _torch()
    lib = _cabi.load()
    assert B.is_cuda and B.dtype == torch.float32 and B.stride(1) == 1 and B.shape[0] == fmt.shape[1]
    arr = (C.c_void_p * len(dest_ptrs))(*[int(p) for p in dest_ptrs])
    with torch.cuda.device(B.device):
        s = fmt.c_struct()
        check(lib.lf_spmm_hyb_f32_bcast(C.byref(s), B.data_ptr(), B.stride(0), arr, len(dest_ptrs), int(ldc),
                                        int(B.shape[1]), _stream_ptr(torch)))


def allgather_rows(C_local, row_begin: int, dest_ptrs: Sequence[int], ldc: int):
    """``lf_allgather_rows``: store this rank's row block into rows ``row_begin ...`` of every full-size
    C whose device address is listed in ``dest_ptrs`` (own buffer and peers' symmetric-memory buffers)."""
    torch = _torch()
    lib = _cabi.load()
    assert C_local.is_cuda and C_local.dtype == torch.float32 and C_local.dim() == 2 and C_local.stride(1) == 1
    arr = (C.c_void_p * len(dest_ptrs))(*[int(p) for p in dest_ptrs])
    with torch.cuda.device(C_local.device):
        check(lib.lf_allgather_rows(C_local.data_ptr(), C_local.stride(0), int(row_begin), int(C_local.shape[0]),
                                    int(C_local.shape[1]), arr, len(dest_ptrs), int(ldc), _stream_ptr(torch)))
