"""Tensor-parallel forward on two GPUs against the CPU restatement (skipped on a single-GPU box)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpus() -> int:
    import torch
    return torch.cuda.device_count()


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["nccl", "peer"])
@pytest.mark.parametrize("key,layers,vocab", [("c5", 2, 4096), ("c2", 2, 4096)])
def test_tensor_parallel_two_gpus(key, layers, vocab, mode):
    if _gpus() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "tp_worker.py"), key, str(layers), str(vocab), "40", "16", mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
