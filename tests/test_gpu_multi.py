"""Column-sharded layer with the gathering epilogue on two or more GPUs (skipped on a single-GPU machine).

The ranks are child processes, one per GPU; NVLS is switched off for every library they load and the kernels use
plain peer stores, so a child that fails cannot disturb the other GPUs' memory mappings.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_gathering_epilogue_across_gpus():
    world = min(torch.cuda.device_count(), 4)
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", "29631", os.path.join(here, "multi_gpu_child.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
