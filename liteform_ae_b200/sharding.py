"""Row sharding over the GPUs of one node (one process per GPU, ``torch.distributed``).

The reference runs on device 0 only (playground_pipline/format_algos.py:548).  Rows of A are
independent in C = A B, so G ranks each own a contiguous, nnz-balanced row range: the bucket
widths are chosen on the whole matrix, every rank builds the slice of the format for its rows
(a contiguous slice of every bucket), B is replicated, and each rank writes only its rows of
C.  The product itself needs no communication; the one collective is the optional all-gather
of the row blocks of C when the caller wants the full matrix on every rank.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np


def split_points_host(indptr: np.ndarray, num_shards: int) -> List[int]:
    """``cuts[g]`` = first row r with ``indptr[r] >= g * nnz / G`` (what ``lf_shard_rows``
    computes on the device); ``cuts[0] = 0``, ``cuts[G] = M``."""
    indptr = np.asarray(indptr, dtype=np.int64)
    M = len(indptr) - 1
    nnz = int(indptr[-1] - indptr[0])
    cuts = [int(np.searchsorted(indptr, int(indptr[0]) + (nnz * g) // num_shards, side="left"))
            for g in range(num_shards)]
    return cuts + [M]


def my_range(cuts: Sequence[int], rank: int) -> Tuple[int, int]:
    return int(cuts[rank]), int(cuts[rank + 1])


def all_gather_rows(C_local, cuts: Sequence[int], group=None):
    """Full ``C`` (``cuts[-1]`` rows) on every rank from the per-rank row blocks.

    Row blocks differ in size, NCCL's all-gather does not take ragged inputs: every rank pads
    its block to the largest one, one ``all_gather`` moves them, and the valid rows are copied
    out.  Works with the ``nccl`` (GPU) and ``gloo`` (CPU tests) back ends.
    """
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    sizes = [int(cuts[g + 1] - cuts[g]) for g in range(world)]
    assert C_local.shape[0] == sizes[rank], "local block does not match the shard plan"
    N = C_local.shape[1]
    biggest = max(sizes)
    padded = C_local
    if sizes[rank] != biggest:
        padded = torch.zeros((biggest, N), dtype=C_local.dtype, device=C_local.device)
        padded[:sizes[rank]] = C_local
    bufs = [torch.empty((biggest, N), dtype=C_local.dtype, device=C_local.device) for _ in range(world)]
    dist.all_gather(bufs, padded.contiguous(), group=group)
    full = torch.empty((int(cuts[-1]), N), dtype=C_local.dtype, device=C_local.device)
    for g in range(world):
        full[cuts[g]:cuts[g + 1]] = bufs[g][:sizes[g]]
    return full


class ShardedSpmm:
    """Per-rank state of a row-sharded SpMM: the rank's slice of the format and its C block."""

    def __init__(self, csr_dev, bucket_widths, rank: int, world: int, cuts: Optional[Sequence[int]] = None):
        from . import hyb
        self.rank, self.world = rank, world
        self.cuts = list(cuts) if cuts is not None else hyb.shard_rows(csr_dev, world)
        self.row_range = my_range(self.cuts, rank)
        self.fmt = hyb.build_hyb_device(csr_dev, bucket_widths, row_range=self.row_range, with_mask=False)

    def spmm(self, B, out=None):
        from . import hyb
        return hyb.spmm_hyb(self.fmt, B, out=out)

    def gather(self, C_local, group=None):
        return all_gather_rows(C_local, self.cuts, group)

    # ---- fused product + all-gather -----------------------------------------------------------
    def prepare_fused_gather(self, N: int, group=None):
        """Allocate the full-size C in symmetric memory (``torch.distributed._symmetric_memory``) and
        exchange the peers' buffer addresses.  Collective: every rank of the group must call it."""
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm
        group = dist.group.WORLD if group is None else group
        dev = self.fmt.device
        self.C_full = symm.empty((self.fmt.shape[0], int(N)), dtype=torch.float32, device=dev)
        self._symm = symm.rendezvous(self.C_full, group)
        self._dest_ptrs = [int(p) for p in self._symm.buffer_ptrs]
        assert len(self._dest_ptrs) == self.world
        return self.C_full

    def gather_peer(self, C_local):
        """The whole C on every rank from the per-rank row blocks, by ``lf_allgather_rows``: every rank
        stores its (ragged) block straight into all full-size buffers over NVLink -- no padding, no
        staging copy.  Needs ``prepare_fused_gather`` (the symmetric-memory buffers)."""
        from . import hyb
        self._symm.barrier()                      # nobody still reads the previous product
        hyb.allgather_rows(C_local, self.row_range[0] if hasattr(self, "row_range") else self.cuts[self.rank],
                           self._dest_ptrs, self.C_full.stride(0))
        self._symm.barrier()                      # every rank's rows have landed everywhere
        return self.C_full

    def spmm_gather_fused(self, B):
        """C = A @ B with the whole product on every rank: the kernel's epilogue stores each row of
        this rank's shard into every rank's full-size C (peer stores over NVLink).  Barriers on the
        symmetric-memory handle order it against the previous readers and the next ones."""
        from . import hyb
        self._symm.barrier()                      # nobody still reads the previous product
        hyb.spmm_hyb_bcast(self.fmt, B, self._dest_ptrs, self.C_full.stride(0))
        self._symm.barrier()                      # every rank's rows have landed everywhere
        return self.C_full


def gpu_numa_node(device_index: int) -> int:
    """NUMA node the GPU hangs off (from the PCI device's sysfs entry), or -1 when it cannot be told."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
        with open(f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node") as f:
            return int(f.read().strip())
    except Exception:
        return -1


_numa_buffers = []   # mappings registered with the CUDA driver stay mapped (and registered) until the process exits


def pinned_empty(shape, dtype, numa_node: int = -1):
    """A pinned (page-locked) host tensor.  With ``numa_node >= 0`` its pages are placed on that NUMA
    node first (anonymous mapping, ``mbind``, first touch) and then registered with the CUDA driver:
    on a two-socket host every GPU then exchanges data with the memory of its own socket instead of
    all GPUs sharing one socket's memory path.  Any failure on that route (no such node, policy not
    permitted in this container) falls back to an ordinary pinned allocation.  Returns
    ``(tensor, placed)``.  A placed buffer is kept mapped and registered for the life of the process
    (an unmapped but still registered range would make a later registration at the same address
    fail); nothing outlasts the process."""
    import ctypes
    import mmap
    import torch
    numel = 1
    for d in shape:
        numel *= int(d)
    nbytes = max(numel * torch.empty((), dtype=dtype).element_size(), 1)
    if numa_node >= 0:
        try:
            size = -(-nbytes // mmap.PAGESIZE) * mmap.PAGESIZE
            buf = mmap.mmap(-1, size)
            addr = ctypes.addressof(ctypes.c_char.from_buffer(buf))
            libc = ctypes.CDLL(None, use_errno=True)
            mask = (ctypes.c_ulong * 16)()
            mask[numa_node // 64] = 1 << (numa_node % 64)
            MPOL_BIND, SYS_MBIND = 2, 237          # x86-64
            rc = libc.syscall(SYS_MBIND, ctypes.c_void_p(addr), ctypes.c_ulong(size), MPOL_BIND, mask,
                              ctypes.c_ulong(16 * 64 + 1), 0)
            if rc != 0:
                raise OSError(ctypes.get_errno(), "mbind")
            ctypes.memset(addr, 0, size)             # first touch: the pages are allocated on the node now
            if int(torch.cuda.cudart().cudaHostRegister(addr, size, 0)) != 0:
                try:      # a failed registration leaves its code as the runtime's "last error": take it out
                    ctypes.CDLL("libcudart.so.12").cudaGetLastError()
                except OSError:
                    pass
                raise RuntimeError("cudaHostRegister")
            _numa_buffers.append(buf)
            t = torch.frombuffer(buf, dtype=torch.uint8, count=nbytes).view(dtype)[:numel].view(*shape)
            return t, True
        except Exception:
            pass
    return torch.empty(tuple(int(d) for d in shape), dtype=dtype).pin_memory(), False


def b_chunk(num_cols: int, world: int, rank: int) -> Tuple[int, int, int]:
    """Rows of B a rank uploads when B starts in host memory: ``(first, last, chunk)`` with equal
    chunks of ``ceil(K / world)`` rows (the last one may be short)."""
    chunk = -(-int(num_cols) // int(world))
    first = min(rank * chunk, num_cols)
    return first, min(first + chunk, num_cols), chunk


class HostShardedSpmm:
    """Row-sharded product whose operands start in HOST memory and whose result returns there.

    Every rank needs all of B.  Uploading it once per rank sends ``world`` copies over the
    host links, which the GPUs of a node share; here each rank uploads only its ``1 / world`` of
    B's rows (``b_chunk``) next to its shard of the format, and one all-gather over NVLink
    completes B on every GPU -- the one exchange step of this path.  Then the device product runs
    and the rank's rows of C go back to the host.  ``slots`` independent sets of device buffers
    and streams let a caller keep several products in flight (the result of one crosses the bus
    while the operands of the next come in); the collectives are issued in call order, so all
    ranks must enqueue the same sequence of slots.
    """

    def __init__(self, fmt, N: int, rank: int, world: int, group=None, slots: int = 2, numa_node: int = -1):
        import copy
        import torch
        self.torch, self.rank, self.world, self.group, self.N = torch, rank, world, group, int(N)
        dev = fmt.device
        self.K = fmt.shape[1]
        self.first, self.last, self.chunk = b_chunk(self.K, world, rank)

        def pin(t):   # host copy of a format array, on the GPU's NUMA node when one is given
            h, _ = pinned_empty(t.shape, t.dtype, numa_node)
            h.copy_(t)
            return h

        names = ("rows", "cols", "vals") + (("zero_rows",) if fmt.num_zero_rows else ())
        self.h_fmt = {n: pin(getattr(fmt, n)) for n in names}
        self.slots = []
        for _ in range(slots):
            f = copy.copy(fmt)
            f.mask = None
            for n in names:
                setattr(f, n, torch.empty_like(getattr(fmt, n)))
            self.slots.append({
                "fmt": f, "stream": torch.cuda.Stream(device=dev),
                "B_chunk": torch.empty((self.chunk, self.N), dtype=torch.float32, device=dev),
                "B_full": torch.empty((self.chunk * world, self.N), dtype=torch.float32, device=dev),
                "C": torch.empty((fmt.row_end - fmt.row_begin, self.N), dtype=torch.float32, device=dev)})
        self.format_bytes = sum(t.numel() * t.element_size() for t in self.h_fmt.values())
        self.h2d_bytes = self.format_bytes + (self.last - self.first) * self.N * 4
        self.d2h_bytes = (fmt.row_end - fmt.row_begin) * self.N * 4

    def enqueue(self, B_rows_host, C_host, slot: int = 0, format_resident: bool = False, events=None):
        """``B_rows_host``: pinned float32 tensor holding THIS rank's rows ``first:last`` of B;
        ``C_host``: pinned float32 tensor for this rank's rows of C.  Returns after enqueueing.
        ``format_resident``: skip the upload of the format when this slot already holds it from an
        earlier call (the reference uploads it on every call, format_algos.py:568-578).
        ``events``: a list that receives five CUDA events recorded on the slot's stream -- start,
        after the uploads, after the all-gather of B, after the product, after the download -- so
        that a caller can tell the phases of one call apart."""
        import torch.distributed as dist
        from . import hyb
        torch, s = self.torch, self.slots[slot]

        def mark():
            if events is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                events.append(ev)

        with torch.cuda.stream(s["stream"]):
            mark()
            if not (format_resident and s.get("has_format")):
                for n, h in self.h_fmt.items():
                    getattr(s["fmt"], n).copy_(h, non_blocking=True)
                s["has_format"] = True
            s["B_chunk"][:self.last - self.first].copy_(B_rows_host, non_blocking=True)
            mark()
            dist.all_gather_into_tensor(s["B_full"], s["B_chunk"], group=self.group)
            mark()
            hyb.spmm_hyb(s["fmt"], s["B_full"][:self.K], out=s["C"])
            mark()
            C_host.copy_(s["C"], non_blocking=True)
            mark()

    def synchronize(self):
        for s in self.slots:
            s["stream"].synchronize()
