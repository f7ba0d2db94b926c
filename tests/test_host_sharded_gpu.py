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
