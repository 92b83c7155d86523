"""Timers, NVTX ranges and the per-step metrics line.

The reference has no tracing or metrics (only glog lines, test/example/test_gpt2.cc:207).  Here:
``nvtx_range`` marks a region for Nsight tools, ``CudaTimer`` measures a region on the device with
CUDA events, ``ThroughputMeter`` turns step times into tokens/s and model FLOP utilisation against
the measured peak, ``JsonlLogger`` appends one JSON object per step to a file, ``annotate_modules``
adds one NVTX range per sub-module, ``PhaseProfiler`` gives the device time of forward / backward /
optimizer phases, and ``torch_profile`` wraps ``torch.profiler`` and writes a Chrome trace.
"""
from __future__ import annotations

import contextlib
import json
import time
from typing import Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class CudaTimer:
    """``with CudaTimer() as t: ...`` then ``t.ms`` (device time between the two events; CPU wall time without CUDA)."""

    def __init__(self, sync: bool = True):
        self.sync, self.ms = sync, 0.0

    def __enter__(self):
        self.cuda = torch.cuda.is_available()
        if self.cuda:
            self.e0, self.e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.e0.record()
        else:
            self.t0 = time.perf_counter()
        return self

    def __exit__(self, *exc):
        if self.cuda:
            self.e1.record()
            if self.sync:
                self.e1.synchronize()
                self.ms = self.e0.elapsed_time(self.e1)
        else:
            self.ms = (time.perf_counter() - self.t0) * 1e3
        return False


class ThroughputMeter:
    def __init__(self, tokens_per_step: int, flops_per_token: float = 0.0, peak_tflops: float = 0.0, n_gpus: int = 1):
        self.tokens, self.fpt, self.peak, self.n = tokens_per_step, flops_per_token, peak_tflops, n_gpus

    def report(self, ms_per_step: float) -> dict:
        tps = self.tokens / (ms_per_step / 1e3)
        out = {"ms_per_step": ms_per_step, "tokens_per_s": tps}
        if self.fpt and self.peak:
            out["mfu"] = tps * self.fpt / (self.peak * 1e12 * self.n)
        return out


class JsonlLogger:
    def __init__(self, path: Optional[str]):
        self.f = open(path, "a") if path else None

    def log(self, **kv) -> None:
        if self.f:
            self.f.write(json.dumps(kv) + "\n")
            self.f.flush()

    def close(self) -> None:
        if self.f:
            self.f.close()


def annotate_modules(model: torch.nn.Module, prefix: str = "") -> list:
    """Wraps every sub-module's forward in an NVTX range named after its dotted path, so that Nsight timelines
    show the model structure.  Returns the hook handles (call ``.remove()`` on each to undo)."""
    handles = []
    if not torch.cuda.is_available():
        return handles
    for name, mod in model.named_modules():
        label = f"{prefix}{name or model.__class__.__name__}"
        handles.append(mod.register_forward_pre_hook(lambda m, a, _l=label: torch.cuda.nvtx.range_push(_l)))
        handles.append(mod.register_forward_hook(lambda m, a, o: torch.cuda.nvtx.range_pop()))
    return handles


class PhaseProfiler:
    """Device time of the phases of a training step (forward, backward, gradient sync, optimizer ...).

        prof = PhaseProfiler()
        with prof.phase("forward"): loss = model(x, y)
        with prof.phase("backward"): loss.backward()
        print(prof.summary())   # {"forward": {"ms": ..., "share": ...}, ...}

    Phases are bracketed by CUDA events on the current stream and read once, in ``summary()``, so the profiled
    loop itself is not synchronised (on CPU the wall clock is used).
    """

    def __init__(self):
        self._events, self._wall = [], []

    @contextlib.contextmanager
    def phase(self, name: str):
        cuda = torch.cuda.is_available()
        with nvtx_range(name):
            if cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            else:
                t0 = time.perf_counter()
            try:
                yield
            finally:
                if cuda:
                    e1.record()
                    self._events.append((name, e0, e1))
                else:
                    self._wall.append((name, (time.perf_counter() - t0) * 1e3))

    def summary(self, reset: bool = True) -> dict:
        tot: dict = {}
        if self._events:
            torch.cuda.synchronize()
        for name, e0, e1 in self._events:
            tot[name] = tot.get(name, 0.0) + e0.elapsed_time(e1)
        for name, ms in self._wall:
            tot[name] = tot.get(name, 0.0) + ms
        total = sum(tot.values()) or 1.0
        if reset:
            self._events, self._wall = [], []
        return {k: {"ms": v, "share": v / total} for k, v in tot.items()}


@contextlib.contextmanager
def torch_profile(trace_path: str, with_stack: bool = False):
    """``torch.profiler`` over a region (CPU + CUDA activities), exported as a Chrome trace to ``trace_path``."""
    from torch.profiler import ProfilerActivity, profile

    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with profile(activities=acts, with_stack=with_stack) as prof:
        yield prof
    prof.export_chrome_trace(trace_path)
