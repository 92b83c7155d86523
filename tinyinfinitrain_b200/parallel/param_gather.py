"""Weights sharded by rows over the data-parallel group, gathered inside the GEMM that consumes them.

ZeRO-style sharding normally ends every step with an all-gather of the updated parameters.  Here that collective
disappears into the next forward pass: every rank keeps a full-size copy of the weight in symmetric memory but is
authoritative only for ``out_features / world`` rows (the rows its optimizer shard updates).  The forward GEMM
(``csrc/kernels/gemm_param_gather.cu``) starts on the n-blocks of the local rows while helper CTAs of the same kernel
pull the other ranks' rows over NVLink into the local copy, chunk by chunk, flag by flag.  After the launch the local
copy is complete, so the backward GEMMs of the step use it as an ordinary operand.

* :class:`GatheredWeightLinear` -- the layer,
* :class:`RowShardedAdam` -- AdamW that reduce-scatters the weight gradients by rows, keeps fp32 master weights and
  moments for the owned rows only and writes the new bf16 rows into the local copy (no parameter broadcast).

Ordering between steps: a rank may overwrite its rows only after every rank has finished the forward GEMM that read
them.  The gradient reduce-scatter of :class:`RowShardedAdam` (a collective every rank enters after its backward pass)
is that fence; the forward GEMM in turn is preceded by a device barrier, which orders it after the owners' updates.

On CPU tensors (gloo groups) the layer all-gathers the rows with ``torch.distributed`` and calls ``F.linear``: the same
semantics, which is what the CPU tests check.  The reference has no data parallelism
(``infini_train/src/device.cc:11-17``).
"""
from __future__ import annotations

import math
from typing import Iterable, Optional

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .. import nn as tnn
from ..ops import functional as ops_f


class _GatheredLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, layer):
        from .._lib import C

        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        layer.barrier()                       # the owners' last updates of their rows are complete and visible
        if b is not None:
            y2 = C.gemm_param_gather(x2, w, layer.peer_row_ptrs, layer.rank, epilogue=ops_f.EPI_BIAS, bias=b,
                                     helper_ctas=layer.helper_ctas)[0]
        else:
            y2 = C.gemm_param_gather(x2, w, layer.peer_row_ptrs, layer.rank, helper_ctas=layer.helper_ctas)[0]
        ctx.save_for_backward(x2, w)
        ctx.b, ctx.xshape = b, x.shape
        return y2.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .._lib import C

        x2, w = ctx.saved_tensors             # w: the local copy, complete since the forward launch
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = C.gemm(dy2, w, False, True)[0].view(ctx.xshape) if ctx.needs_input_grad[0] else None
        dw = ops_f._wgrad(dy2, x2, w) if ctx.needs_input_grad[1] else None
        db = ops_f._bgrad(dy2, ctx.b) if (ctx.b is not None and ctx.needs_input_grad[2]) else None
        return dx, dw, db, None


class GatheredWeightLinear(tnn.Module):
    """``y = x W^T + b`` with ``W [out, in]`` sharded by rows over ``group``.

    ``weight`` is this rank's full-size copy (a view of symmetric memory on CUDA); rows
    ``[rank * rows_per_rank, (rank + 1) * rows_per_rank)`` are the ones this rank owns.  ``out_features`` must be a
    multiple of ``128 * world`` on CUDA (128-row chunks per owner)."""

    kType = "Linear"
    kParamWeightName = "weight"
    kParamBiasName = "bias"

    def __init__(self, in_features: int, out_features: int, bias: bool = True, group: Optional[dist.ProcessGroup] = None,
                 device=None, dtype=torch.bfloat16, helper_ctas: int = 0, channel: int = 3):
        super().__init__()
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.in_features, self.out_features, self.helper_ctas = in_features, out_features, helper_ctas
        if out_features % self.world:
            raise ValueError("GatheredWeightLinear: out_features must divide over the group")
        self.rows_per_rank = out_features // self.world
        dev = torch.device(device if device is not None else "cpu")
        self.fused = dev.type == "cuda"
        if self.fused:
            from .symm import DeviceBarrier, SymmetricBuffer

            if dtype != torch.bfloat16 or self.rows_per_rank % 128 or in_features % 8:
                raise ValueError("GatheredWeightLinear on CUDA: bf16, 128-row chunks per rank, in_features % 8 == 0")
            self.buf = SymmetricBuffer(out_features * in_features, dtype, dev, self.group)
            storage = self.buf.tensor
            self.barrier = DeviceBarrier(self.buf, channel=channel)
            esize = storage.element_size()
            self.peer_row_ptrs = [int(p) + r * self.rows_per_rank * in_features * esize for r, p in enumerate(self.buf.ptrs)]
        else:
            storage = torch.empty(out_features * in_features, dtype=dtype, device=dev)
            self.buf, self.barrier, self.peer_row_ptrs = None, (lambda: None), []
        self.weight = torch.nn.Parameter(storage.view(out_features, in_features))
        self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=dtype, device=dev)) if bias else None
        self.reset_parameters()

    def own_rows(self) -> slice:
        return slice(self.rank * self.rows_per_rank, (self.rank + 1) * self.rows_per_rank)

    @torch.no_grad()
    def reset_parameters(self, seed: int = 42) -> None:
        """Same values on every rank (seeded), like a replicated layer after the initial broadcast; rows a rank
        does not own are then deliberately scrambled on CUDA, so that a forward pass that failed to gather them
        cannot go unnoticed."""
        g = torch.Generator().manual_seed(seed)
        bound = 1.0 / math.sqrt(self.in_features)
        full = (torch.rand(self.out_features, self.in_features, generator=g) * 2 - 1) * bound
        self.weight.copy_(full.to(self.weight.dtype))
        if self.bias is not None:
            self.bias.copy_(((torch.rand(self.out_features, generator=g) * 2 - 1) * bound).to(self.bias.dtype))
        if self.fused:
            keep = self.weight[self.own_rows()].clone()
            self.weight.fill_(float("nan"))
            self.weight[self.own_rows()] = keep
            torch.cuda.synchronize(self.weight.device)
            dist.barrier(group=self.group)

    def ResetParameters(self) -> None:
        self.reset_parameters()

    def forward(self, x):
        if self.fused:
            return _GatheredLinearFn.apply(x, self.weight, self.bias, self)
        # CPU: gather the rows through the process group, then an ordinary linear on the refreshed local copy
        with torch.no_grad():
            mine = self.weight[self.own_rows()].contiguous()
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
            self.weight.copy_(torch.cat(parts))
        return F.linear(x, self.weight, self.bias)


class RowShardedAdam:
    """AdamW for :class:`GatheredWeightLinear` layers (plus any replicated parameters).

    Weight gradients are reduce-scattered by rows (rank r receives the summed gradient of the rows it owns), the fp32
    master rows and moments live on the owner only, and the new bf16 rows are written into the owner's local copy --
    no parameter all-gather: the next forward GEMM fetches them.  Replicated parameters (biases, anything passed in
    ``replicated``) get an all-reduced gradient and the full update on every rank."""

    def __init__(self, layers: Iterable[GatheredWeightLinear], replicated: Iterable[torch.nn.Parameter] = (), lr: float = 1e-3,
                 betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0, group: Optional[dist.ProcessGroup] = None):
        self.layers = list(layers)
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.t = 0
        self.rows = []
        for l in self.layers:
            w = l.weight.detach()[l.own_rows()].float().clone()
            self.rows.append({"master": w, "m": torch.zeros_like(w), "v": torch.zeros_like(w)})
        self.replicated = [p for l in self.layers if l.bias is not None for p in [l.bias]] + list(replicated)
        self.rep = [{"master": p.detach().float().clone(), "m": torch.zeros_like(p, dtype=torch.float32),
                     "v": torch.zeros_like(p, dtype=torch.float32)} for p in self.replicated]

    @property
    def params(self):
        return [l.weight for l in self.layers] + self.replicated

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            p.grad = None

    ZeroGrad = zero_grad

    def _adam(self, st, g) -> None:
        b1, b2 = self.betas
        st["m"].mul_(b1).add_(g, alpha=1 - b1)
        st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
        mh, vh = st["m"] / (1 - b1 ** self.t), st["v"] / (1 - b2 ** self.t)
        st["master"].sub_(self.lr * (mh / (vh.sqrt() + self.eps) + self.weight_decay * st["master"]))

    @torch.no_grad()
    def step(self) -> None:
        self.t += 1
        for l, st in zip(self.layers, self.rows):
            g = l.weight.grad
            if g is None:
                g = torch.zeros_like(l.weight)
            g = g.float().contiguous()
            if g.is_cuda:
                shard = torch.empty_like(st["master"])
                dist.reduce_scatter_tensor(shard.view(-1), g.view(-1), op=dist.ReduceOp.SUM, group=self.group)
            else:                              # gloo has no reduce-scatter
                dist.all_reduce(g, group=self.group)
                shard = g[l.own_rows()]
            self._adam(st, shard / self.world)
            l.weight[l.own_rows()] = st["master"].to(l.weight.dtype)
        for p, st in zip(self.replicated, self.rep):
            g = (p.grad if p.grad is not None else torch.zeros_like(p)).float()
            dist.all_reduce(g, group=self.group)
            self._adam(st, g / self.world)
            p.copy_(st["master"].to(p.dtype))

    Step = step
