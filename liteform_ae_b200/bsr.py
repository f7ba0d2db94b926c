"""Block-sparse (8x8 BSR) matrices in device memory and their SpMM.

The reference converts the graph with SciPy (``MTX.tobsr_with_padding``,
playground_pipline/format_matrix_market.py:116-138, block size 32, fp16) and times a generated
wmma kernel (``bench_bsrmm``, playground_pipline/format_algos.py:1562-1643).  Here the format
stays SciPy's (``indptr``, sorted ``indices``, dense ``data[nb, R, C]``), cut into 8x8 tiles on
the device when it comes in coarser, and the product runs on ``lf_spmm_bsr8_{f32,bf16,f16}``.
``DeviceBsr8.from_csr_device`` converts a CSR matrix that already lies in device memory.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import numpy as np

from . import _cabi
from ._cabi import check, t_ptr
from .timing import profile_ms


def _torch():
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("liteform_ae_b200 needs a CUDA device (there is no CPU path)")
    return torch


@dataclass
class DeviceBsr8:
    indptr: "object"        # torch int64 [Mb + 1]
    indices: "object"       # torch int32 [nb]
    blocks: "object"        # torch float32 / bfloat16 / float16 [nb, 8, 8]
    shape: Tuple[int, int]

    @property
    def num_blocks(self) -> int:
        return int(self.indices.numel())

    @staticmethod
    def from_arrays(indptr, indices, blocks, shape, dtype="float32", device="cuda") -> "DeviceBsr8":
        torch = _torch()
        assert blocks.ndim == 3 and blocks.shape[1:] == (8, 8), "blocks must be [nb, 8, 8]"
        assert shape[0] % 8 == 0 and shape[1] % 8 == 0, "matrix dimensions must be multiples of 8"
        tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}[str(dtype)]
        b = torch.from_numpy(np.ascontiguousarray(blocks, dtype=np.float32)).to(device).to(tdt).contiguous()
        return DeviceBsr8(torch.from_numpy(np.ascontiguousarray(indptr, dtype=np.int64)).to(device),
                          torch.from_numpy(np.ascontiguousarray(indices, dtype=np.int32)).to(device),
                          b, (int(shape[0]), int(shape[1])))

    @staticmethod
    def from_csr_device(csr, dtype="float32", padded_shape: Optional[Tuple[int, int]] = None) -> "DeviceBsr8":
        """CSR in device memory (``hyb.DeviceCsr``) -> 8x8 blocks, without leaving the device
        (``lf_bsr8_plan`` + ``lf_bsr8_fill``).  ``padded_shape`` (multiples of 8, at least the
        matrix shape) plays the role of the ``shape`` argument of ``MTX.tobsr_with_padding``
        (format_matrix_market.py:116-138); by default each dimension is rounded up to 8."""
        torch = _torch()
        lib = _cabi.load()
        import ctypes
        M, K = csr.shape
        M8, K8 = (-(-M // 8) * 8, -(-K // 8) * 8) if padded_shape is None else map(int, padded_shape)
        assert M8 % 8 == 0 and K8 % 8 == 0 and M8 >= M and K8 >= K, "padded shape must be multiples of 8 covering the matrix"
        dev = csr.indptr.device
        tdt, code = {"float32": (torch.float32, _cabi.LF_DTYPE_F32), "bfloat16": (torch.bfloat16, _cabi.LF_DTYPE_BF16),
                     "float16": (torch.float16, _cabi.LF_DTYPE_F16)}[str(dtype)]
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream().cuda_stream
            indptr8 = torch.empty(M8 // 8 + 1, dtype=torch.int64, device=dev)
            nb = ctypes.c_int64(0)
            check(lib.lf_bsr8_plan(t_ptr(csr.indptr), t_ptr(csr.indices), M, t_ptr(indptr8), ctypes.byref(nb), stream))
            Mb = -(-M // 8)
            if M8 // 8 > Mb:                       # block rows that exist only as padding
                indptr8[Mb + 1:] = indptr8[Mb]
            indices8 = torch.empty(nb.value, dtype=torch.int32, device=dev)
            blocks = torch.empty((nb.value, 8, 8), dtype=tdt, device=dev)
            check(lib.lf_bsr8_fill(t_ptr(csr.indptr), t_ptr(csr.indices), t_ptr(csr.data) if csr.data is not None else None,
                                   M, t_ptr(indptr8), t_ptr(indices8), t_ptr(blocks), code, stream))
        return DeviceBsr8(indptr8, indices8, blocks, (M8, K8))

    @staticmethod
    def from_scipy(bsr_mat, dtype: Optional[str] = None, device="cuda") -> "DeviceBsr8":
        """Accepts a ``scipy.sparse.bsr_matrix`` with blocks whose sides are multiples of 8 on a shape
        that is a multiple of the block size.  The block arrays are uploaded as they are; blocks
        coarser than 8x8 (the reference passes 32x32, format_algos.py:1562-1643) are cut into 8x8
        tiles on the device and all-zero tiles dropped (``lf_bsr_split8_plan`` / ``_fill``) -- the
        result equals ``scipy.sparse.bsr_matrix(blocksize=(8, 8))`` of the matrix without its
        explicit zeros."""
        torch = _torch()
        lib = _cabi.load()
        import ctypes
        m = bsr_mat
        if dtype is None:
            dtype = "float16" if m.data.dtype == np.float16 else "float32"
        R, Cb = m.blocksize
        assert R % 8 == 0 and Cb % 8 == 0, "block size must be a multiple of 8"
        assert m.shape[0] % R == 0 and m.shape[1] % Cb == 0, "shape must be a multiple of the block size"
        m_indptr, m_indices, m_data = m.indptr, m.indices, m.data
        row_of = np.repeat(np.arange(len(m_indptr) - 1), np.diff(m_indptr))
        if m_indices.size and not (np.diff(m_indices)[np.diff(row_of) == 0] > 0).all():
            # block columns must ascend inside a block row (SciPy's own sort refuses float16 data)
            order = np.lexsort((m_indices, row_of))
            m_indices, m_data = m_indices[order], m_data[order]
        in_np = {np.dtype(np.float16): (np.float16, torch.float16, _cabi.LF_DTYPE_F16)}.get(
            m_data.dtype, (np.float32, torch.float32, _cabi.LF_DTYPE_F32))
        tdt, out_code = {"float32": (torch.float32, _cabi.LF_DTYPE_F32), "bfloat16": (torch.bfloat16, _cabi.LF_DTYPE_BF16),
                         "float16": (torch.float16, _cabi.LF_DTYPE_F16)}[str(dtype)]
        block_rows, nb = m.shape[0] // R, int(m_indices.shape[0])
        indptr = torch.from_numpy(np.ascontiguousarray(m_indptr, dtype=np.int64)).to(device)
        indices = torch.from_numpy(np.ascontiguousarray(m_indices, dtype=np.int32)).to(device)
        data = torch.from_numpy(np.ascontiguousarray(m_data, dtype=in_np[0])).to(device)
        dev = indptr.device
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream().cuda_stream
            sc_bytes = lib.lf_bsr_split8_scratch_bytes(nb, R, Cb)
            scratch = torch.empty(sc_bytes, dtype=torch.uint8, device=dev)
            fine_rows = block_rows * (R // 8)
            indptr8 = torch.empty(fine_rows + 1, dtype=torch.int64, device=dev)
            n_tiles = ctypes.c_int64(0)
            check(lib.lf_bsr_split8_plan(t_ptr(indptr), t_ptr(data), in_np[2], block_rows, nb, R, Cb, t_ptr(scratch),
                                         sc_bytes, t_ptr(indptr8), ctypes.byref(n_tiles), stream))
            indices8 = torch.empty(n_tiles.value, dtype=torch.int32, device=dev)
            blocks = torch.empty((n_tiles.value, 8, 8), dtype=tdt, device=dev)
            check(lib.lf_bsr_split8_fill(t_ptr(indptr), t_ptr(indices), t_ptr(data), in_np[2], block_rows, nb, R, Cb,
                                         t_ptr(scratch), t_ptr(indptr8), t_ptr(indices8), t_ptr(blocks), out_code, stream))
            torch.cuda.current_stream().synchronize()      # scratch and the coarse arrays are released on return
        return DeviceBsr8(indptr8, indices8, blocks, (int(m.shape[0]), int(m.shape[1])))


def spmm_bsr8(a: DeviceBsr8, B, out=None, block_row_range=None):
    """C = A @ B for an 8x8-block matrix; B's dtype must match the blocks', C is float32."""
    torch = _torch()
    lib = _cabi.load()
    assert B.is_cuda and B.dim() == 2 and B.stride(1) == 1 and B.shape[0] == a.shape[1]
    assert B.dtype == a.blocks.dtype, "B and the blocks must have the same dtype"
    r0, r1 = (0, a.shape[0] // 8) if block_row_range is None else block_row_range
    N = int(B.shape[1])
    if out is None:
        out = torch.empty(((r1 - r0) * 8, N), dtype=torch.float32, device=B.device)
    assert out.dtype == torch.float32 and out.shape == ((r1 - r0) * 8, N) and out.stride(1) == 1
    fn = {torch.float32: lib.lf_spmm_bsr8_f32, torch.bfloat16: lib.lf_spmm_bsr8_bf16,
          torch.float16: lib.lf_spmm_bsr8_f16}[a.blocks.dtype]
    with torch.cuda.device(B.device):
        check(fn(t_ptr(a.indptr), t_ptr(a.indices), t_ptr(a.blocks), r0, r1, B.data_ptr(), B.stride(0),
                 out.data_ptr(), out.stride(0), N, torch.cuda.current_stream().cuda_stream))
    return out


def bench_bsrmm(bsr_mat, x, block_size, device="cuda", warmup=10, repeat=100) -> float:
    """Drop-in for the reference's ``bench_bsrmm(bsr_mat, x, block_size)``: uploads the matrix and
    x, runs the block SpMM and returns its mean time in milliseconds (format_algos.py:1562-1643).
    fp16 inputs (what the reference passes) run with fp32 accumulation."""
    torch = _torch()
    assert bsr_mat.blocksize == (block_size, block_size), "block_size does not match the matrix"
    a = DeviceBsr8.from_scipy(bsr_mat, device=device)
    xt = x if isinstance(x, torch.Tensor) else torch.as_tensor(np.asarray(x))
    xt = xt.to(device=device, dtype=a.blocks.dtype).contiguous()
    out = spmm_bsr8(a, xt)
    dur = profile_ms(lambda: spmm_bsr8(a, xt, out=out), warmup=warmup, repeat=repeat)
    print("bsrmm exe time: {:.6f} ms".format(dur))
    return dur
