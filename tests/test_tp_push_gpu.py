"""Tensor-parallel decode on two GPUs of one box: the exchange fused into the GEMV epilogue (peer
stores + polling reduce) against the NCCL allreduce and against the unsharded engine.  Skipped on
a box with fewer than two GPUs; NVLS is switched off for NCCL, the push uses plain peer stores."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_push_exchange_matches_unsharded_engine_on_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    worker = Path(__file__).with_name("tp_push_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                           "--master-port", "29577", str(worker)], env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    assert "push vs unsharded" in done.stdout
