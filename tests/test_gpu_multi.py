"""Sharded configurations on two or more GPUs of one box (skipped on a single-GPU box): one
process per GPU launched with torch.distributed.run, NCCL through the C ABI."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_tp_and_ep_on_two_gpus(cuda):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"  # plain peer paths only: a rank that dies on a failed check must not hold a multicast binding
    port = 29600 + os.getpid() % 1000
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "multi_gpu_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "rank 0 ok" in proc.stdout and "rank 1 ok" in proc.stdout
