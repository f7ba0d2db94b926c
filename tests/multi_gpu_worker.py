"""One rank of the multi-GPU test (started by tests/test_multi_gpu.py under torch.distributed.run).

Every rank builds its nnz-balanced row shard of a seeded matrix, then produces the WHOLE product on
every GPU three ways -- fused epilogue (lf_spmm_hyb_f32_bcast: peer stores and peer vector atomics
from inside the product kernel), product + lf_allgather_rows (ragged peer-store gather), product +
padded NCCL all-gather -- and compares each with SciPy in float64 (rel 1e-5 / abs 1e-4).  Also
runs the host-operand path (sharding.HostShardedSpmm) once.  Rank 0 prints "MULTI_GPU_OK <world>"."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    from liteform_ae_b200 import hyb, synth, width_search
    from liteform_ae_b200.sharding import HostShardedSpmm, ShardedSpmm
    from oracle import hyb_oracle as ho

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    try:
        for name, make, N, P in (("skew", lambda: synth.skewed_rows(M=8192, seed=3), 64, 1),
                                 ("powerlaw", lambda: synth.power_law_graph(M=16384, seed=1), 128, 2)):
            csr = make()
            d = hyb.DeviceCsr.from_host(csr.indptr, csr.indices, csr.data, csr.shape, dev)
            stats, hist = hyb.hyb_stats(d, P)
            widths = width_search.search_from_stats(stats, hist, N, P)
            sh = ShardedSpmm(d, widths, rank, world)
            B = synth.dense_features(csr.shape[1], N, 5)
            Bd = torch.from_numpy(B).to(dev)
            want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data.astype(np.float64), csr.shape, B.astype(np.float64))
            sh.prepare_fused_gather(N)
            for rep in range(2):     # twice: the buffers are reused, the barriers must order the rounds
                full = sh.spmm_gather_fused(Bd)
                np.testing.assert_allclose(full.cpu().numpy(), want, rtol=1e-5, atol=1e-4, err_msg=f"fused {name}")
            local_C = sh.spmm(Bd)
            full = sh.gather_peer(local_C)
            np.testing.assert_allclose(full.cpu().numpy(), want, rtol=1e-5, atol=1e-4, err_msg=f"peer gather {name}")
            full = sh.gather(local_C)
            np.testing.assert_allclose(full.cpu().numpy(), want, rtol=1e-5, atol=1e-4, err_msg=f"nccl gather {name}")
            if P == 1:
                hs = HostShardedSpmm(sh.fmt, N, rank, world, slots=2)
                B_rows = torch.from_numpy(B[hs.first:hs.last]).pin_memory()
                Cp = [torch.full((sh.row_range[1] - sh.row_range[0], N), float("nan")).pin_memory() for _ in range(2)]
                for k in (0, 1, 0, 1):
                    hs.enqueue(B_rows, Cp[k], k, format_resident=True)
                hs.synchronize()
                for k in (0, 1):
                    np.testing.assert_allclose(Cp[k].numpy(), want[sh.row_range[0]:sh.row_range[1]], rtol=1e-5, atol=1e-4)
            dist.barrier()
        if rank == 0:
            print(f"MULTI_GPU_OK {world}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
