"""The example entry points on CPU: one process, and gloo ranks for tensor / pipeline / data parallel layouts."""
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
COMMON = ["--device", "cpu", "--synthetic", "--num_iteration", "3", "--n_layer", "2", "--batch_size", "2",
          "--sequence_length", "16", "--dtype", "float32"]


def _losses(out: str):
    return [float(m) for m in re.findall(r"^step \d+/\d+ \| loss ([0-9.]+)", out, flags=re.M)]


def _sane(ls, vocab):
    """Every step sees fresh random tokens, so the loss stays near ln(vocab); it must be finite and reported thrice."""
    import math

    return len(ls) == 3 and all(math.isfinite(x) and abs(x - math.log(vocab)) < 2.0 for x in ls)


def _run(cmd):
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


@pytest.mark.parametrize("family", ["gpt2", "llama3"])
def test_single_process_training_runs(family):
    out = _run([sys.executable, f"examples/{family}/main.py"] + COMMON)
    assert _sane(_losses(out), 50257 if family == "gpt2" else 128256), out[-1500:]


@pytest.mark.parametrize("layout", [["--tensor_parallel", "2", "--pipeline_parallel", "2", "--num_microbatches", "2"],
                                    ["--tensor_parallel", "2"],                       # tp2 x dp2 with ZeRO-1
                                    ["--pipeline_parallel", "4", "--num_microbatches", "4", "--n_layer", "4"]])
def test_four_ranks_layouts(layout):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
           "127.0.0.1", "--master-port", str(29250 + os.getpid() % 200), "examples/gpt2/main.py"] + COMMON + layout
    out = _run(cmd)
    assert _sane(_losses(out), 50257), out[-1500:]
