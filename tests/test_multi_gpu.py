"""Peer paths on real GPUs: the fused product + all-gather (lf_spmm_hyb_f32_bcast), the ragged peer
gather (lf_allgather_rows) and the host-operand path, with one process per GPU over NCCL.  Needs two
devices; the ranks run tests/multi_gpu_worker.py and compare with SciPy themselves."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_whole_product_on_every_gpu_three_ways(cuda_device):
    import torch
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    res = subprocess.run(cmd, capture_output=True, text=True, env=env, cwd=ROOT, timeout=600)
    assert res.returncode == 0, (res.stdout[-2000:], res.stderr[-4000:])
    assert f"MULTI_GPU_OK {world}" in res.stdout
