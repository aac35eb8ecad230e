"""Multi-GPU checks (NVLink all-reduce, tensor- and expert-parallel layer): spawned as one
process per GPU over 2, 4 or 8 of the visible GPUs (the largest of those that fits)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_all_ranks_allreduce_tp_ep():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    ngpu = torch.cuda.device_count()
    if ngpu < 2:
        pytest.skip("needs at least two GPUs")
    world = 8 if ngpu >= 8 else (4 if ngpu >= 4 else 2)
    # NVLS off: nothing here uses multicast objects, and a rank that failed while bound to one has
    # raised NVLink faults on its peers
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(ROOT, "tests", "multi_gpu_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("multi-GPU checks passed") == world
