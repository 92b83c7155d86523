"""Pipeline parallelism: contiguous stage partition and the 1F1B schedule.

Stage ``s`` of ``P`` runs ``min(P - s - 1, m)`` warm-up forwards, then alternates one forward with
one backward, then drains the remaining backwards, so at most ``P - s`` micro-batch activations
are alive per stage.  Activations and their gradients travel between neighbouring stages with
NCCL point-to-point operations (``batch_isend_irecv``), which run on NCCL's own stream: the send
of micro-batch i overlaps the compute of micro-batch i+1, and only the tensor actually needed
next is waited for.  With sequence parallelism the tensor exchanged is the token shard
``[B*T/tp, C]``, i.e. each tensor-parallel rank talks to its peer in the next stage.

The reference has no pipeline parallelism: ``Sequential`` runs every block in one process
(infini_train/src/nn/modules/container.cc:18-22).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def partition_layers(n_layer: int, pp: int) -> List[range]:
    """Contiguous, balanced split of ``n_layer`` blocks over ``pp`` stages (earlier stages get the remainder)."""
    base, rem = divmod(n_layer, pp)
    out, start = [], 0
    for s in range(pp):
        n = base + (1 if s < rem else 0)
        out.append(range(start, start + n))
        start += n
    return out


def one_f_one_b_order(stage: int, num_stages: int, num_micro: int) -> List[Tuple[str, int]]:
    """The sequence of ('F', i) / ('B', i) steps a stage executes (pure function, used by tests)."""
    warm = min(num_stages - stage - 1, num_micro)
    order: List[Tuple[str, int]] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    for _ in range(num_micro - warm):
        order.append(("F", f)); f += 1
        order.append(("B", b)); b += 1
    while b < num_micro:
        order.append(("B", b)); b += 1
    return order


class PipelineStage:
    """Runs one stage of a 1F1B pipeline.

    ``forward_fn(x_in, micro_index) -> tensor``: the stage's computation.  On the first stage
    ``x_in`` is None (the function reads its own input batch); on the last stage the returned
    tensor is the scalar loss of the micro-batch, on the others the activation for the next stage.
    """

    def __init__(self, forward_fn: Callable, stage: int, num_stages: int, prev_rank: Optional[int],
                 next_rank: Optional[int], act_shape: Sequence[int], dtype: torch.dtype, device,
                 group: Optional[dist.ProcessGroup] = None):
        self.fn, self.stage, self.P = forward_fn, stage, num_stages
        self.prev, self.next = prev_rank, next_rank
        self.shape, self.dtype, self.device, self.group = tuple(act_shape), dtype, device, group
        self.first, self.last = stage == 0, stage == num_stages - 1

    # ---- point-to-point helpers -------------------------------------------------------------------
    def _exchange(self, send_next=None, send_prev=None, recv_prev=False, recv_next=False):
        ops, rp, rn = [], None, None
        if send_prev is not None:
            ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), self.prev, self.group))
        if recv_prev:
            rp = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, rp, self.prev, self.group))
        if send_next is not None:
            ops.append(dist.P2POp(dist.isend, send_next.contiguous(), self.next, self.group))
        if recv_next:
            rn = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, rn, self.next, self.group))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return rp, rn

    # ---- one training step over `num_micro` micro-batches --------------------------------------------
    def run(self, num_micro: int) -> Optional[torch.Tensor]:
        """Executes the 1F1B schedule; returns the mean micro-batch loss on the last stage, else None."""
        inputs: List[Optional[torch.Tensor]] = []
        outputs: List[torch.Tensor] = []
        losses: List[torch.Tensor] = []
        warm = min(self.P - self.stage - 1, num_micro)
        steady = num_micro - warm
        fi = 0

        def forward(x_in):
            nonlocal fi
            if x_in is not None:
                x_in.requires_grad_(True)
            out = self.fn(x_in, fi)
            fi += 1
            if self.last:
                losses.append(out.detach())
                out = out / num_micro
            inputs.append(x_in)
            outputs.append(out)
            return out

        def backward(dout):
            x_in, out = inputs.pop(0), outputs.pop(0)
            if self.last:
                out.backward()
            else:
                torch.autograd.backward(out, dout)
            return None if x_in is None else x_in.grad

        x = None
        for _ in range(warm):
            if not self.first:
                x, _ = self._exchange(recv_prev=True)
            out = forward(x)
            if not self.last:
                self._exchange(send_next=out.detach())
        if steady > 0 and not self.first:
            x, _ = self._exchange(recv_prev=True)
        for i in range(steady):
            out = forward(x)
            dout = None
            if not self.last:
                _, dout = self._exchange(send_next=out.detach(), recv_next=True)
            dx = backward(dout)
            last_iter = i == steady - 1
            if not self.first:
                if last_iter:
                    self._exchange(send_prev=dx)
                else:
                    x, _ = self._exchange(send_prev=dx, recv_prev=True)
        for _ in range(warm):
            dout = None
            if not self.last:
                _, dout = self._exchange(recv_next=True)
            dx = backward(dout)
            if not self.first:
                self._exchange(send_prev=dx)
        if self.last:
            return torch.stack(losses).mean()
        return None
