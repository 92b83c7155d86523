"""Profiling helpers on CPU: phase timing, throughput / MFU arithmetic, JSONL sink, Chrome trace export."""
import json
import time

import torch

from tinyinfinitrain_b200.utils import JsonlLogger, PhaseProfiler, ThroughputMeter, annotate_modules, torch_profile


def test_phase_profiler_accumulates_and_resets():
    prof = PhaseProfiler()
    for _ in range(2):
        with prof.phase("forward"):
            time.sleep(0.01)
        with prof.phase("backward"):
            time.sleep(0.02)
    s = prof.summary()
    assert set(s) == {"forward", "backward"}
    assert s["backward"]["ms"] > s["forward"]["ms"] >= 15
    assert abs(s["forward"]["share"] + s["backward"]["share"] - 1.0) < 1e-9
    assert prof.summary() == {}


def test_throughput_and_mfu():
    m = ThroughputMeter(tokens_per_step=8192, flops_per_token=6 * 124e6, peak_tflops=1000.0, n_gpus=2)
    r = m.report(10.0)
    assert r["tokens_per_s"] == 819200.0
    assert abs(r["mfu"] - 819200.0 * 6 * 124e6 / (1000e12 * 2)) < 1e-12


def test_jsonl_logger_and_trace(tmp_path):
    log = JsonlLogger(str(tmp_path / "m.jsonl"))
    log.log(step=1, loss=2.5)
    log.log(step=2, loss=2.0)
    log.close()
    rows = [json.loads(x) for x in open(tmp_path / "m.jsonl")]
    assert rows == [{"step": 1, "loss": 2.5}, {"step": 2, "loss": 2.0}]
    lin = torch.nn.Linear(4, 4)
    assert annotate_modules(lin) == [] or torch.cuda.is_available()
    with torch_profile(str(tmp_path / "trace.json")):
        lin(torch.randn(2, 4)).sum().backward()
    assert "traceEvents" in json.load(open(tmp_path / "trace.json"))


def test_warmup_cosine_schedule_and_scheduler():
    import math

    from tinyinfinitrain_b200.optim import LRScheduler, warmup_cosine

    f = lambda s: warmup_cosine(s, 1.0, 4, 20, 0.1)  # noqa: E731
    assert [round(f(s), 4) for s in range(4)] == [0.25, 0.5, 0.75, 1.0]
    assert f(4) == 1.0 and abs(f(12) - (0.1 + 0.9 * 0.5)) < 1e-12 and abs(f(20) - 0.1) < 1e-12 and f(1000) == 0.1
    assert all(f(s) >= f(s + 1) for s in range(4, 25))
    assert abs(warmup_cosine(8, 2.0, 0, 16, 0.0) - 2.0 * 0.5 * (1 + math.cos(math.pi / 2))) < 1e-12

    class Opt:
        lr = 0.0

        def set_lr(self, lr):
            self.lr = lr

    o = Opt()
    sched = LRScheduler(o, f)
    assert o.lr == 0.25
    assert [sched.step() for _ in range(3)] == [0.5, 0.75, 1.0] and o.lr == 1.0
