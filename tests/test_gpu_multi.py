"""Multi-GPU tests: each launches torchrun workers, one rank per GPU (skipped with fewer than 2 GPUs)."""
import os
import subprocess
import sys

import pytest
import torch

from _launch import run_group

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _torchrun(script, nproc, extra_env=None, timeout=600):
    env = dict(os.environ, **(extra_env or {}))
    port = 29600 + os.getpid() % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, script)]
    return run_group(cmd, env=env, timeout=timeout)


def _ngpu():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_zero1_fused_matches_nccl():
    r = _torchrun("dist_zero_check.py", min(_ngpu(), 8))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(_ngpu() < 2, reason="needs 2 GPUs")
def test_tp_fused_collectives_match_nccl():
    n = 2 if _ngpu() < 4 else 4 if _ngpu() < 8 else 8
    r = _torchrun("dist_tp_check.py", n)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-3000:]
