"""Training-step driver: static buffers, optional CUDA-graph capture of the whole step.

``TrainStep`` is the public entry point a training loop (and ``bench.py``) calls:
one call copies a batch from pinned host memory, runs forward + backward + gradient
synchronisation + optimizer on the device, and returns the loss in pinned host memory.
With ``use_graph=True`` the device work of one step is captured once in a CUDA graph
and replayed, which removes every per-kernel launch cost from the loop; all
step-dependent scalars (Adam step count, learning rate) live in device memory so the
replayed graph stays correct.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch


class TrainStep:
    def __init__(self, model, optimizer, batch_size: int, seq_len: int, device, use_graph: bool = True,
                 grad_sync: Optional[Callable[[], None]] = None, loss_scale: float = 1.0):
        self.model, self.opt = model, optimizer
        self.device = torch.device(device)
        self.use_graph = use_graph and self.device.type == "cuda"
        self.grad_sync = grad_sync
        self.idx = torch.zeros(batch_size, seq_len, dtype=torch.int64, device=self.device)
        self.tgt = torch.zeros(batch_size, seq_len, dtype=torch.int64, device=self.device)
        self.loss = torch.zeros((), dtype=torch.float32, device=self.device)
        pin = self.device.type == "cuda"
        self.host_loss = torch.zeros((), dtype=torch.float32, pin_memory=pin)
        self.graph = None
        self.launches_per_step = 0

    def _device_step(self) -> None:
        self.opt.zero_grad()
        _, loss = self.model(self.idx, self.tgt, return_logits=False)
        loss.backward()
        if self.grad_sync is not None:
            self.grad_sync()
        self.opt.step()
        self.loss.copy_(loss.detach().float())

    def prepare(self, eager_warmup: int = 2) -> None:
        """Runs a few eager steps (first-use allocations, attribute set-up) and captures the graph."""
        from .._lib import C

        if self.device.type != "cuda":
            return
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            for i in range(max(1, eager_warmup)):
                before = C.launch_count()
                self._device_step()
                self.launches_per_step = C.launch_count() - before
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        if self.use_graph:
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                self._device_step()
            torch.cuda.synchronize(self.device)

    def run_device(self) -> None:
        """Device work of one step on the current stream (inputs already in the static buffers)."""
        if self.graph is not None:
            self.graph.replay()
        else:
            self._device_step()

    def __call__(self, idx_host: torch.Tensor, tgt_host: torch.Tensor) -> torch.Tensor:
        """One end-to-end step; returns the pinned host scalar (valid after a stream sync)."""
        self.idx.copy_(idx_host, non_blocking=True)
        self.tgt.copy_(tgt_host, non_blocking=True)
        self.run_device()
        self.host_loss.copy_(self.loss, non_blocking=True)
        return self.host_loss
