"""The library's exchange over NVLink peer memory on two or more GPUs (skipped on a single-GPU machine): one process per
GPU, launched the way the benchmark is launched."""
import os
import subprocess
import sys

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_memory_exchange_matches_gathered_sums():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
                        "--master-port", "29611", os.path.join(ROOT, "tests", "multi_gpu_worker.py")], capture_output=True, text=True, timeout=600,
                       env=env)
    assert r.returncode == 0 and "MULTI_GPU_WORKER_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
