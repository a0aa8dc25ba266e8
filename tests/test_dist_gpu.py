"""The multi-GPU operators of att3ntion_b200._dist with the real kernels: one process per GPU over NCCL, every
rank's shard against the whole problem computed on its own GPU (Y and dQ bit-identical, key gradients to FP32
summation order).  Needs at least two GPUs; the host logic alone is covered on CPU by tests/test_dist_cpu.py."""
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
WORKER = Path(__file__).resolve().parent / "helpers" / "dist_gpu_worker.py"


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="requires two CUDA devices")
def test_row_and_head_sharding_with_the_kernels():
    world = min(torch.cuda.device_count(), 4)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                        "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(WORKER)],
                       capture_output=True, text=True, timeout=600,
                       env={**__import__("os").environ, "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0 and f"dist-gpu-ok {world}" in r.stdout, (r.stdout[-2000:], r.stderr[-4000:])
