"""Sharded configurations on two or more GPUs of one box (skipped on a single-GPU box): one
process per GPU launched with torch.distributed.run, NCCL through the C ABI for set-up, this
library's kernels over NVLink peer memory for the sums and the expert exchange.  Run at 2 ranks and,
where the box has them, at 4 and 8."""
import os
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
def test_tp_and_ep_on_several_gpus(cuda, world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"  # plain peer paths only: a rank that dies on a failed check must not hold a multicast binding
    port = 29600 + (os.getpid() + world) % 1000
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world), "--master-addr",
           "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / "multi_gpu_worker.py")]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    for r in range(world):
        assert f"rank {r} ok" in proc.stdout
