"""bench.py's control flow and output contract, dry-run on CPU (tiny model, gloo ranks, wall-clock timing)."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REQUIRED = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
            "vs_baseline", "dtype", "data", "config", "clocks", "e2e", "gpu_launches", "impl"}


def _run(cmd, timeout=600):
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def _check(out, n, impl):
    assert REQUIRED <= set(out), REQUIRED - set(out)
    assert out["n_gpus"] == n and out["steps"] == 2 and out["warmup"] >= 3 and out["impl"] == impl
    assert out["value"] > 0 and out["higher_is_better"] is True and out["scaling"] == "weak"
    assert out["config"]["global_batch"] == 2 * n and out["config"]["seq_len"] == 32
    e = out["e2e"]
    assert e["value"] > 0 and e["h2d_bytes_per_step"] == 2 * 2 * 32 * 8 and e["d2h_bytes_per_step"] == 4
    assert set(out["clocks"]) >= {"sm_mhz", "sm_max_mhz", "reasons"}


def test_bench_single_rank_dry_run():
    args = ["--device", "cpu", "--tiny", "--steps", "2", "--warmup", "1", "--batch", "2", "--seq", "32"]
    _check(_run([sys.executable, "bench.py"] + args), 1, "ours")
    _check(_run([sys.executable, "bench.py", "--impl", "library"] + args), 1, "library")


def test_bench_two_ranks_dry_run():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(29800 + os.getpid() % 100), "bench.py", "--gpus", "2", "--device", "cpu",
           "--tiny", "--steps", "2", "--warmup", "3", "--batch", "2", "--seq", "32"]
    _check(_run(cmd), 2, "ours")


def test_reference_arm_reports_unavailable():
    r = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1"],
                       cwd=ROOT, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["impl"] == "reference" and "unavailable" in out and "\n" not in out["unavailable"]


def test_pipeline_bubble_bench_two_stages_dry_run():
    """utils/pp_bench.py on two gloo ranks: the record carries the measured and the ideal bubble of the 1F1B schedule."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(29700 + os.getpid() % 100), "-m", "tinyinfinitrain_b200.utils.pp_bench",
           "--micro", "2", "--batch", "1", "--seq", "32", "--layers", "2", "--d_model", "64", "--heads", "2", "--iters", "2"]
    out = _run(cmd)
    assert out["stages"] == 2 and out["micro_batches"] == 2 and out["ms_2m"] > 0 and out["ms_m"] > 0
    assert abs(out["bubble_ideal"] - 1.0 / 3.0) < 1e-9 and abs(out["bubble_ideal_2m"] - 0.2) < 1e-9
    assert abs(out["slot_ms"] * 2 - (out["ms_2m"] - out["ms_m"])) < 1e-6


import pytest  # noqa: E402


@pytest.mark.parametrize("config,parallelism", [("llama1b_tp8", "tp8+sp+dp1"), ("gpt2xl_tp2pp2dp2", "tp2+sp+pp2+dp2+zero1"),
                                                ("llama8b_tp4dp2", "tp4+sp+dp2+zero1")])
def test_bench_named_eight_rank_layouts_dry_run(config, parallelism):
    """The three 8-GPU configurations of the bench with their real process layout (tensor x pipeline x data parallel
    groups, sequence parallelism, ZeRO-1, 1F1B micro-batches) on eight gloo ranks and a tiny model of the same family."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "8", "--master-addr",
           "127.0.0.1", "--master-port", str(29600 + os.getpid() % 100), "bench.py", "--gpus", "8", "--device", "cpu",
           "--tiny", "--config", config, "--steps", "2", "--warmup", "3", "--batch", "2", "--seq", "32", "--micro", "2",
           "--no-baseline"]
    out = _run(cmd, timeout=900)
    assert out["n_gpus"] == 8 and out["config"]["name"] == config and out["config"]["parallelism"] == parallelism
    assert out["value"] > 0 and out["scaling"] == "strong" and out["config"]["final_loss"] > 0
