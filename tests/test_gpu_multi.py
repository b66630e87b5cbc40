"""Runs tests/multi_gpu_gates.py on the GPUs of the box (needs at least two): the reduce inside the kernel
for tensor-parallel and for expert-parallel ranks, the latter with ragged expert counts."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gates(n, port, *extra):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "multi_gpu_gates.py"), *extra]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "MULTI-GPU GATES: PASS" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_fused_tensor_parallel_gates():
    n = 4 if torch.cuda.device_count() >= 4 else 2
    _gates(n, 29533, "--parallel", "tp", "--tokens", "8192", "--ncomm", "14")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_fused_expert_parallel_gates_with_ragged_counts():
    n = 8 if torch.cuda.device_count() >= 8 else (4 if torch.cuda.device_count() >= 4 else 2)
    _gates(n, 29534, "--parallel", "ep", "--tokens", "8192,16384", "--ncomm", "14,32", "--skew", "1.0", "--soak", "12",
           "--soak-tokens", "2048,4096")
