"""Multi-rank host logic on CPU: shard planning and the ragged all-gather over gloo (world 2, 3)."""
import os
import socket

import numpy as np
import pytest

from oracle import hyb_oracle as ho
from liteform_ae_b200 import sharding, synth


def test_split_points_balance_nnz():
    csr = synth.skewed_rows(M=4096, seed=2, heavy_rows=4, heavy_len=500)
    for G in (1, 2, 3, 8):
        cuts = sharding.split_points_host(csr.indptr, G)
        assert cuts[0] == 0 and cuts[-1] == 4096 and all(a <= b for a, b in zip(cuts, cuts[1:]))
        nnz = np.diff(csr.indptr[cuts])
        longest = int(np.diff(csr.indptr).max())
        assert nnz.sum() == csr.nnz and nnz.max() <= csr.nnz / G + longest
    # degenerate: more shards than rows with entries
    tiny = synth.Csr(np.array([0, 0, 3, 3], dtype=np.int64), np.array([0, 1, 2], dtype=np.int32),
                     np.ones(3, np.float32), (3, 3))
    cuts = sharding.split_points_host(tiny.indptr, 4)
    assert cuts[0] == 0 and cuts[-1] == 3 and all(a <= b for a, b in zip(cuts, cuts[1:]))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        csr = synth.zipf_rows(M=1500, seed=4)
        B = synth.dense_features(1500, 16, 0)
        cuts = sharding.split_points_host(csr.indptr, world)
        a, b = sharding.my_range(cuts, rank)
        sub = csr.toscipy()[a:b]
        C_local = torch.from_numpy(np.asarray(sub @ B))
        full = sharding.all_gather_rows(C_local, cuts)
        want = ho.spmm_scipy_csr(csr.indptr, csr.indices, csr.data, csr.shape, B)
        ok = bool(np.array_equal(full.numpy(), want))
        q.put((rank, ok, tuple(full.shape)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_all_gather_rows_gloo(world):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == list(range(world))
    assert all(r[1] for r in results), results


def test_b_chunks_cover_all_rows_once():
    from liteform_ae_b200.sharding import b_chunk
    for K, world in ((1 << 20, 8), (1000, 3), (7, 8), (1, 1), (4096, 5)):
        spans = [b_chunk(K, world, r) for r in range(world)]
        assert all(c == spans[0][2] for _, _, c in spans) and spans[0][2] * world >= K
        covered = np.zeros(K, dtype=int)
        for r, (a, b, c) in enumerate(spans):
            assert 0 <= a <= b <= K and b - a <= c and a == min(r * c, K)
            covered[a:b] += 1
        assert (covered == 1).all()
