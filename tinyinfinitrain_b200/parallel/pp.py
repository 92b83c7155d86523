"""Pipeline parallelism: contiguous stage partition and the 1F1B schedule.

Stage ``s`` of ``P`` runs ``min(P - s - 1, m)`` warm-up forwards, then alternates one forward with
one backward, then drains the remaining backwards, so at most ``P - s`` micro-batch activations
are alive per stage.  Activations and their gradients travel between neighbouring stages with
NCCL point-to-point operations (``batch_isend_irecv``), which run on NCCL's own stream: a batch
that only sends is not waited for inside the schedule (the next micro-batch is launched at once and
the handles are drained at the end of the step), the receives of the warm-up and cool-down phases
are posted one micro-batch ahead, and a receive is waited for where its tensor is first used.  With sequence parallelism the tensor exchanged is the token shard
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
        self.trace = None        # set to a list to record ("issue" | "wait", kind) and ("F" | "B", micro-batch) events
        self._deferred = []

    # ---- point-to-point helpers -------------------------------------------------------------------
    # Every transfer is a NCCL / gloo point-to-point operation issued through ``batch_isend_irecv``; a send and a
    # receive that go to the same neighbour at the same point of the schedule travel in ONE batch (two separate
    # operations towards one peer could each wait for the other side's matching call and deadlock).  What differs is
    # when the compute stream waits:
    #   * a receive is waited for at the point where its tensor is first used, and the receives of the warm-up and
    #     cool-down phases (where no send goes to that neighbour) are posted one micro-batch ahead;
    #   * a batch that only sends is never waited for inside the schedule: the next forward / backward is launched
    #     right away and the handles are drained once at the end of the step (the sent tensors are kept alive until
    #     then).  A batch that sends and receives is waited for because of its receive.
    def _issue(self, send_next=None, send_prev=None, recv_prev=False, recv_next=False):
        """Posts the transfers; returns (handles, recv_prev_buffer, recv_next_buffer, kept_tensors)."""
        ops, rp, rn, keep = [], None, None, []
        if send_prev is not None:
            t = send_prev.contiguous()
            keep.append(t)
            ops.append(dist.P2POp(dist.isend, t, self.prev, self.group))
        if recv_prev:
            rp = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, rp, self.prev, self.group))
        if send_next is not None:
            t = send_next.contiguous()
            keep.append(t)
            ops.append(dist.P2POp(dist.isend, t, self.next, self.group))
        if recv_next:
            rn = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, rn, self.next, self.group))
        works = dist.batch_isend_irecv(ops) if ops else []
        kind = ("s" if keep else "") + ("r" if (recv_prev or recv_next) else "")
        self._log("issue", kind)
        return works, rp, rn, keep

    def _wait(self, works, kind="r"):
        self._log("wait", kind)
        for w in works:
            w.wait()

    def _send_only(self, send_next=None, send_prev=None):
        works, _, _, keep = self._issue(send_next=send_next, send_prev=send_prev)
        self._deferred.append((works, keep))

    def _drain(self):
        for works, _keep in self._deferred:
            self._wait(works, "s")
        self._deferred = []

    def _log(self, *event):
        if self.trace is not None:
            self.trace.append(event)

    # ---- one training step over `num_micro` micro-batches --------------------------------------------
    def run(self, num_micro: int) -> Optional[torch.Tensor]:
        """Executes the 1F1B schedule; returns the mean micro-batch loss on the last stage, else None."""
        inputs: List[Optional[torch.Tensor]] = []
        outputs: List[torch.Tensor] = []
        losses: List[torch.Tensor] = []
        warm = min(self.P - self.stage - 1, num_micro)
        steady = num_micro - warm
        fi = 0
        self._deferred = []

        def forward(x_in):
            nonlocal fi
            self._log("F", fi)
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

        bi = 0

        def backward(dout):
            nonlocal bi
            self._log("B", bi)
            bi += 1
            x_in, out = inputs.pop(0), outputs.pop(0)
            if self.last:
                out.backward()
            else:
                torch.autograd.backward(out, dout)
            return None if x_in is None else x_in.grad

        # ---- warm-up: forwards only.  The input of forward i+1 is requested before forward i is computed.
        x, pending = None, None
        n_fwd_inputs = (warm + (1 if steady > 0 else 0)) if not self.first else 0   # receives before the steady phase
        if n_fwd_inputs > 0:
            pending = self._issue(recv_prev=True)
        for i in range(warm):
            if not self.first:
                works, x, _, _ = pending
                pending = self._issue(recv_prev=True) if i + 1 < n_fwd_inputs else None
                self._wait(works)
            out = forward(x)
            if not self.last:
                self._send_only(send_next=out.detach())
        if steady > 0 and not self.first:
            works, x, _, _ = pending
            self._wait(works)
        # ---- steady state: one forward, one backward; each exchange pairs a send with the receive it enables
        for i in range(steady):
            out = forward(x)
            dout = None
            if not self.last:
                works, _, dout, keep = self._issue(send_next=out.detach(), recv_next=True)
                self._wait(works, "sr")
            dx = backward(dout)
            last_iter = i == steady - 1
            if not self.first:
                if last_iter:
                    self._send_only(send_prev=dx)
                else:
                    works, x, _, keep = self._issue(send_prev=dx, recv_prev=True)
                    self._wait(works, "sr")
        # ---- cool-down: backwards only.  The gradient of backward i+1 is requested before backward i runs.
        pending = self._issue(recv_next=True) if (warm > 0 and not self.last) else None
        for i in range(warm):
            dout = None
            if not self.last:
                works, _, dout, _ = pending
                pending = self._issue(recv_next=True) if i + 1 < warm else None
                self._wait(works)
            dx = backward(dout)
            if not self.first:
                self._send_only(send_prev=dx)
        self._drain()
        if self.last:
            return torch.stack(losses).mean()
        return None
