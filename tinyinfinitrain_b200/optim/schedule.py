"""Learning-rate schedules.  The reference trains at a constant rate (a literal in its test fixture,
test/example/test_gpt2.cc:119); these helpers return the rate for a step and push it into an optimizer with
``set_lr``.  The mixed-precision and distributed optimizers keep the rate in device memory, so a training step that was
captured in a CUDA graph picks the new value up on its next replay."""
from __future__ import annotations

import math


def constant(step: int, lr: float) -> float:
    return lr


def warmup_cosine(step: int, max_lr: float, warmup_steps: int, total_steps: int, min_ratio: float = 0.1) -> float:
    """Linear warm-up from 0 over ``warmup_steps`` (step counts from 0), then cosine decay to ``min_ratio * max_lr`` at
    ``total_steps``, constant afterwards (the llm.c / GPT-3 recipe)."""
    if warmup_steps > 0 and step < warmup_steps:
        return max_lr * (step + 1) / warmup_steps
    if step >= total_steps:
        return max_lr * min_ratio
    span = max(1, total_steps - warmup_steps)
    t = (step - warmup_steps) / span
    return max_lr * (min_ratio + (1.0 - min_ratio) * 0.5 * (1.0 + math.cos(math.pi * t)))


class LRScheduler:
    """``sched = LRScheduler(opt, lambda s: warmup_cosine(s, 3e-4, 100, 10000)); sched.step()`` once per optimizer step."""

    def __init__(self, optimizer, fn):
        self.opt, self.fn, self.t = optimizer, fn, 0
        self._apply()

    def _apply(self) -> None:
        lr = float(self.fn(self.t))
        if hasattr(self.opt, "set_lr"):
            self.opt.set_lr(lr)
        else:
            self.opt.lr = lr
        self.lr = lr

    def step(self) -> float:
        self.t += 1
        self._apply()
        return self.lr
