"""Timers, NVTX ranges and the per-step metrics line.

The reference has no tracing or metrics (only glog lines, test/example/test_gpt2.cc:207).  Here:
``nvtx_range`` marks a region for Nsight tools, ``CudaTimer`` measures a region on the device with
CUDA events, ``ThroughputMeter`` turns step times into tokens/s and model FLOP utilisation against
the measured peak, and ``JsonlLogger`` appends one JSON object per step to a file.
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
