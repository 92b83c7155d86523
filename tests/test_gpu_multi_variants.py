"""Multi-GPU jobs (2+ GPUs, child processes under torchrun): bucketed ZeRO-1 overlap, fused gradient clipping, the
standalone symmetric-memory collectives against NCCL, the package's own symmetric heap."""
import os
import subprocess
import sys

import pytest
import torch

from _launch import run_group
from tinyinfinitrain_b200 import ops
from tinyinfinitrain_b200._lib import C

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16
HERE = os.path.dirname(os.path.abspath(__file__))


def _multi_rank_env(**extra):
    """Environment of a multi-rank child job: NVLink multicast stays off in NCCL and in this package's kernels
    (plain peer loads / stores), so that a rank that stops early -- a Python error in a new branch, say -- never
    leaves memory bound to a multicast object behind.  TITB_TEST_MULTIMEM=1 runs the multicast branches instead."""
    env = dict(os.environ, **extra)
    if os.environ.get("TITB_TEST_MULTIMEM") != "1":
        env.update(NCCL_NVLS_ENABLE="0", TITB200_NO_MULTIMEM="1", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    else:
        env.update(TITB200_MULTIMEM="1")
    return env



@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_zero1_bucketed_overlap_matches_single_bucket():
    n = min(torch.cuda.device_count(), 8)
    env = _multi_rank_env(TITB_TEST_ZERO_BUCKETS="3")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29900 + os.getpid() % 90), os.path.join(HERE, "dist_zero_check.py")]
    r = run_group(cmd, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_zero1_fused_gradient_clipping_matches_nccl():
    n = min(torch.cuda.device_count(), 8)
    env = _multi_rank_env(TITB_TEST_ZERO_CLIP="0.5")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29850 + os.getpid() % 90), os.path.join(HERE, "dist_zero_check.py")]
    r = run_group(cmd, env=env, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_symmetric_collectives_match_nccl():
    n = min(torch.cuda.device_count(), 8)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29750 + os.getpid() % 90), os.path.join(HERE, "dist_collectives_check.py")]
    r = run_group(cmd, env=_multi_rank_env(), timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_zero1_on_the_native_symmetric_heap():
    """The ZeRO-1 worker with buffers from this package's own heap (cuMem VMM + descriptor passing) instead of
    PyTorch's symmetric-memory allocator."""
    n = min(torch.cuda.device_count(), 8)
    env = _multi_rank_env(TITB200_SYMM_HEAP="native")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr",
           "127.0.0.1", "--master-port", str(29990 - os.getpid() % 90), os.path.join(HERE, "dist_zero_check.py")]
    r = run_group(cmd, env=env, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]

