"""sharding.HostShardedSpmm on one GPU (a process group of one rank over NCCL): operands from
pinned host memory, B completed by the all-gather, result back in host memory; two products in
flight on the two slots."""
import numpy as np
import pytest

from oracle import hyb_oracle as ho
from liteform_ae_b200 import hyb, synth, width_search
from liteform_ae_b200.sharding import HostShardedSpmm

pytestmark = pytest.mark.gpu


@pytest.fixture
def one_rank_group(cuda_device):
    import torch
    import torch.distributed as dist
    if dist.is_initialized():
        pytest.skip("a process group is already active in this process")
    import socket
    with socket.socket() as sock:                      # a port nobody uses right now
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    torch.cuda.set_device(cuda_device)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=0, world_size=1)
    yield
    dist.destroy_process_group()


def test_products_from_host_operands(cuda_device, one_rank_group):
    import torch
    N = 64
    csr = synth.power_law_graph(M=8192, seed=1)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    stats, hist = hyb.hyb_stats(d, 1)
    fmt = hyb.build_hyb_device(d, width_search.search_from_stats(stats, hist, N, 1), with_mask=False)
    hs = HostShardedSpmm(fmt, N, rank=0, world=1, slots=2)
    assert (hs.first, hs.last) == (0, csr.shape[1])
    Bs = [synth.dense_features(csr.shape[1], N, seed) for seed in (3, 4)]
    hB = [torch.from_numpy(b).pin_memory() for b in Bs]
    hC = [torch.full((csr.shape[0], N), float("nan")).pin_memory() for _ in range(2)]
    for rep in range(2):
        for k in (0, 1):
            hs.enqueue(hB[k], hC[k], slot=k)
    hs.synchronize()
    for k in (0, 1):
        want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, Bs[k].astype(np.float64))
        np.testing.assert_allclose(hC[k].numpy(), want, rtol=1e-5, atol=1e-4)


def test_pinned_buffer_on_the_gpus_numa_node(cuda_device):
    """sharding.pinned_empty: pages bound to a NUMA node and registered with the driver (or, where the
    host does not allow that, an ordinary pinned allocation): either way a pinned tensor that asynchronous
    copies in both directions accept, and HostShardedSpmm gives the same product with it."""
    import torch
    from liteform_ae_b200.sharding import gpu_numa_node, pinned_empty
    node = gpu_numa_node(cuda_device.index or 0)
    for want_node in (node if node >= 0 else 0, -1, 4095):        # 4095: no such node -> falls back
        t, placed = pinned_empty((1000, 33), torch.float32, want_node)
        assert t.shape == (1000, 33) and t.dtype == torch.float32 and t.is_pinned()
        assert placed in (True, False) and (want_node >= 0 or not placed)
        x = torch.randn((1000, 33), device=cuda_device)
        t.copy_(x, non_blocking=True)
        torch.cuda.synchronize(cuda_device)
        assert torch.equal(t, x.cpu())
        y = torch.empty_like(x)
        y.copy_(t, non_blocking=True)
        torch.cuda.synchronize(cuda_device)
        assert torch.equal(y, x)


def test_products_from_numa_placed_host_operands(cuda_device, one_rank_group):
    import torch
    from liteform_ae_b200.sharding import gpu_numa_node, pinned_empty
    N = 32
    csr = synth.zipf_rows(M=4096, seed=4)
    d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, cuda_device)
    stats, hist = hyb.hyb_stats(d, 1)
    fmt = hyb.build_hyb_device(d, width_search.search_from_stats(stats, hist, N, 1), with_mask=False)
    node = max(gpu_numa_node(cuda_device.index or 0), 0)
    hs = HostShardedSpmm(fmt, N, rank=0, world=1, slots=2, numa_node=node)
    B = synth.dense_features(csr.shape[1], N, 9)
    hB, _ = pinned_empty(B.shape, torch.float32, node)
    hB.copy_(torch.from_numpy(B))
    hC, _ = pinned_empty((csr.shape[0], N), torch.float32, node)
    for _ in range(2):
        hs.enqueue(hB, hC, slot=0, format_resident=True)
    hs.synchronize()
    want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, B.astype(np.float64))
    np.testing.assert_allclose(hC.numpy(), want, rtol=1e-5, atol=1e-4)
