"""Tensor parallelism with Megatron-style sequence parallelism.

Between tensor-parallel regions activations are sharded over tokens: a rank holds rows
``[r * M/tp, (r+1) * M/tp)`` of the flattened ``[M = B*T, C]`` activation.  A
``ColumnParallelLinear`` all-gathers those rows and multiplies by its slice of the output
features; a ``RowParallelLinear`` multiplies by its slice of the input features and
reduce-scatters the partial sums back to token shards.  The two hot pairs

    all-gather -> GEMM            (column parallel forward, row parallel dgrad)
    GEMM -> reduce-scatter        (row parallel forward, column parallel dgrad)

go through :class:`TPComm`, which either composes NCCL collectives with the tcgen05 GEMM
(``mode="nccl"``, the unfused baseline) or calls the fused kernels of
``csrc/kernels/gemm_collective.cu`` (``mode="fused"``), where peer copies, tensor-core tiles
and the reduction run in one launch over NVLink peer memory.

The reference has no tensor parallelism (its only linear layer is nn::Linear,
infini_train/include/nn/modules/linear.h:11-24).
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from .. import nn, ops
from ..nn import init
from ..ops import functional as F_
from .._lib import C

_bf16 = torch.bfloat16


class TPComm:
    """Communication context of one tensor-parallel group."""

    def __init__(self, group: Optional[dist.ProcessGroup], mode: str = "nccl"):
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.mode = mode if self.world > 1 else "none"
        self._fused = None
        if self.mode == "fused":
            from .fused_tp import FusedTP

            self._fused = FusedTP(self)

    def new_step(self) -> None:
        if self._fused is not None:
            self._fused.new_step()

    # ---- unfused collectives on row-sharded 2-D tensors --------------------------------------
    def all_gather_rows(self, x_s: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x_s
        out = torch.empty(x_s.shape[0] * self.world, *x_s.shape[1:], device=x_s.device, dtype=x_s.dtype)
        if x_s.is_cuda:
            dist.all_gather_into_tensor(out, x_s.contiguous(), group=self.group)
        else:
            parts = list(out.chunk(self.world, 0))
            dist.all_gather(parts, x_s.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, z: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return z
        n = z.shape[0] // self.world
        if z.is_cuda:
            out = torch.empty(n, *z.shape[1:], device=z.device, dtype=z.dtype)
            dist.reduce_scatter_tensor(out, z.contiguous(), group=self.group)
            return out
        zz = z.clone()
        dist.all_reduce(zz, group=self.group)
        return zz[self.rank * n:(self.rank + 1) * n].clone()

    def all_reduce(self, t: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(t, op=op, group=self.group)
        return t

    # ---- statistics exchange of the vocabulary-parallel loss -------------------------------------
    def vp_stats_table(self, rows: int, dev):
        """Returns (table, destination addresses, slot) for the pass-1 kernel of the vocabulary-parallel cross
        entropy.  Fused mode: the table lives in symmetric memory and the kernel stores straight into every
        peer's copy.  NCCL mode: a one-slot local table that :meth:`vp_stats_publish` all-gathers."""
        if self._fused is not None:
            table, ptrs = self._fused.stats_table(rows, dev)
            return table, ptrs, self.rank
        table = torch.empty(1, rows, 3, device=dev, dtype=torch.float32)
        return table, [table.data_ptr()], 0

    def vp_stats_publish(self, table: torch.Tensor, rows: int) -> torch.Tensor:
        if self._fused is not None:
            self._fused.stats_publish(rows, table.device)
            return table
        if self.world == 1:
            return table
        full = torch.empty(self.world, rows, 3, device=table.device, dtype=torch.float32)
        dist.all_gather_into_tensor(full, table, group=self.group)
        return full

    # ---- the two fused pairs ---------------------------------------------------------------------
    def ag_input(self, like: torch.Tensor):
        """Where the producer of the next ``ag_gemm`` operand (same shape and dtype as ``like``) may write its result
        so that no staging copy is needed: a view of the symmetric gather buffer in fused mode, else ``None``."""
        if self._fused is None or not like.is_cuda or like.dtype != _bf16 or like.dim() != 2:
            return None
        return self._fused.ag_input(like.shape[0], like.shape[1], like.device)

    def ag_gemm(self, x_s, w, bias=None, gelu=False, b_mn=False):
        """X = all_gather(x_s); returns (X W^T (+bias) [, pre-activation], X).
        b_mn: ``w`` is stored [K, N] (the product is X W), used by dgrad."""
        if self._fused is not None and x_s.is_cuda and x_s.dtype == _bf16:
            return self._fused.ag_gemm(x_s, w, bias, gelu, b_mn)
        X = self.all_gather_rows(x_s)
        return _local_gemm(X, w, bias, gelu, b_mn) + (X,)

    def gemm_rs(self, y, w, b_mn=False, bias=None, residual_s=None):
        """reduce_scatter_rows(y . W^T) (+bias +residual on the shard).  b_mn: W stored [K, N]."""
        if self._fused is not None and y.is_cuda and y.dtype == _bf16:
            return self._fused.gemm_rs(y, w, b_mn, bias, residual_s)
        if y.is_cuda and y.dtype == _bf16:
            Z = C.gemm(y, w, False, b_mn)[0]
        else:
            Z = y @ (w if b_mn else w.t())
        z_s = self.reduce_scatter_rows(Z)
        if bias is not None:
            z_s = z_s + bias
        if residual_s is not None:
            z_s = z_s + residual_s
        return z_s


def _local_gemm(X, w, bias, gelu, b_mn=False):
    if X.is_cuda and X.dtype == _bf16:
        if gelu:
            act, pre = C.gemm(X, w, False, b_mn, epilogue=F_.EPI_BIAS_GELU, bias=bias, want_aux_out=True)
            return act, pre
        if bias is not None:
            return (C.gemm(X, w, False, b_mn, epilogue=F_.EPI_BIAS, bias=bias)[0],)
        return (C.gemm(X, w, False, b_mn)[0],)
    Y = X @ (w if b_mn else w.t())
    if bias is not None:
        Y = Y + bias
    if gelu:
        return ops.gelu_ref(Y), Y
    return (Y,)


def _wgrad_any(dy2, x2, w):
    if dy2.is_cuda and dy2.dtype == _bf16:
        return F_._wgrad(dy2, x2, w)
    return dy2.t() @ x2


def _bgrad_any(dy2, b):
    if dy2.is_cuda and dy2.dtype in (_bf16, torch.float32):
        return F_._bgrad(dy2.contiguous(), b)
    return dy2.sum(0)


class _ColumnParallelFn(torch.autograd.Function):
    """x_s [M/tp, K] -> Y [M, N/tp] = all_gather(x_s) W^T + b."""

    @staticmethod
    def forward(ctx, x_s, w, b, comm: TPComm):
        Y, X = comm.ag_gemm(x_s, w, b)
        ctx.save_for_backward(X, w)
        ctx.b, ctx.comm = b, comm
        return Y

    @staticmethod
    def backward(ctx, dY):
        X, w = ctx.saved_tensors
        comm = ctx.comm
        dY = dY.contiguous()
        dx_s = comm.gemm_rs(dY, w, b_mn=True)          # (dY W) reduce-scattered to token shards
        dw = _wgrad_any(dY, X, w)
        db = _bgrad_any(dY, ctx.b) if ctx.b is not None else None
        return dx_s, dw, db, None


class _RowParallelFn(torch.autograd.Function):
    """y [M, K/tp] -> z_s [M/tp, N] = reduce_scatter(y W^T) + b + residual_s."""

    @staticmethod
    def forward(ctx, y, w, b, residual_s, comm: TPComm):
        z_s = comm.gemm_rs(y, w, False, b, residual_s)
        ctx.save_for_backward(y, w)
        ctx.b, ctx.comm, ctx.has_res = b, comm, residual_s is not None
        return z_s

    @staticmethod
    def backward(ctx, dz_s):
        y, w = ctx.saved_tensors
        comm = ctx.comm
        dz_s = dz_s.contiguous()
        # dY = all_gather(dz_s) . W ; the gathered dZ comes back as a by-product for the wgrad
        dY, dZ = comm.ag_gemm(dz_s, w, b_mn=True)
        dw = _wgrad_any(dZ, y, w)
        db = _bgrad_any(dz_s, ctx.b) if ctx.b is not None else None
        return dY, dw, db, (dz_s if ctx.has_res else None), None


class _TPMLPGeluFn(torch.autograd.Function):
    """Sequence-parallel GPT-2 MLP: x_s -> all-gather -> GEMM(+bias+GELU) -> GEMM -> reduce-scatter (+bias+residual)."""

    @staticmethod
    def forward(ctx, x_s, w1, b1, w2, b2, residual_s, comm: TPComm):
        act, pre, X = comm.ag_gemm(x_s, w1, b1, gelu=True)
        z_s = comm.gemm_rs(act, w2, False, b2, residual_s)
        ctx.save_for_backward(X, w1, w2, pre, act)
        ctx.b1, ctx.b2, ctx.comm, ctx.has_res = b1, b2, comm, residual_s is not None
        return z_s

    @staticmethod
    def backward(ctx, dz_s):
        X, w1, w2, pre, act = ctx.saved_tensors
        comm = ctx.comm
        dz_s = dz_s.contiguous()
        dact, dZ = comm.ag_gemm(dz_s, w2, b_mn=True)
        if pre.is_cuda and pre.dtype == _bf16:
            dpre = C.gelu_bwd(dact, pre)
        else:
            p = pre.detach().requires_grad_(True)
            with torch.enable_grad():
                ops.gelu_ref(p).backward(dact)
            dpre = p.grad
        dw2 = _wgrad_any(dZ, act, w2)
        db2 = _bgrad_any(dz_s, ctx.b2) if ctx.b2 is not None else None
        dx_s = comm.gemm_rs(dpre, w1, b_mn=True)
        dw1 = _wgrad_any(dpre, X, w1)
        db1 = _bgrad_any(dpre, ctx.b1) if ctx.b1 is not None else None
        return dx_s, dw1, db1, dw2, db2, (dz_s if ctx.has_res else None), None


def _mark_sp(p: torch.nn.Parameter) -> torch.nn.Parameter:
    """Parameters replicated across the tensor-parallel group but fed token shards (norm weights,
    row-parallel biases, position embeddings) see only their shard's gradient: it is summed over
    the group before the optimizer step (see ``sync_sequence_parallel_grads``)."""
    p._sp_grad_sync = True
    return p


def sync_sequence_parallel_grads(params, comm: TPComm) -> None:
    """Sums the gradients of the parameters that are replicated over the tensor-parallel group (each rank saw only its
    token shard).  When the parameters live in a flat buffer (``optim.FlatParams`` puts the replicated ones first) the
    whole region is reduced by one collective; parameters outside a flat buffer are reduced one by one."""
    if comm.world == 1:
        return
    done = set()
    for p in params:
        if not getattr(p, "_sp_grad_sync", False):
            continue
        flat = getattr(p, "_flat", None)
        if flat is not None and getattr(p, "main_grad", None) is not None:
            if id(flat) not in done and flat.n_replicated > 0:
                # a replicated parameter without a gradient this step must not contribute stale values
                for q in flat.params:
                    if getattr(q, "_sp_grad_sync", False) and q._fresh_grad and q.grad is None:
                        q.main_grad.zero_()
                        q._fresh_grad = False
                    elif getattr(q, "_sp_grad_sync", False) and q.grad is not None:
                        (q.main_grad.copy_ if q._fresh_grad else q.main_grad.add_)(q.grad)
                        q._fresh_grad, q.grad = False, None
                comm.all_reduce(flat.grad[:flat.n_replicated])
                done.add(id(flat))
            continue
        g = getattr(p, "main_grad", None)
        if g is None:
            g = p.grad
        if g is not None:
            comm.all_reduce(g)


class ColumnParallelLinear(nn.Module):
    """Linear layer whose output features are split over the tensor-parallel group.

    Input: token shard ``[M/tp, in]``.  Output: ``[M, out/tp]`` (all tokens, local features).
    """

    kType = "ColumnParallelLinear"

    def __init__(self, in_features: int, out_features: int, comm: TPComm, bias: bool = True, device=None,
                 dtype=torch.float32, out_local: Optional[int] = None):
        super().__init__()
        assert out_local is not None or out_features % comm.world == 0
        self.comm, self.in_features, self.out_features = comm, in_features, out_features
        self.out_local = out_local if out_local is not None else out_features // comm.world  # uneven splits pass it
        self.weight = torch.nn.Parameter(torch.empty(self.out_local, in_features, device=device, dtype=dtype))
        self.bias = torch.nn.Parameter(torch.zeros(self.out_local, device=device, dtype=dtype)) if bias else None
        init.KaimingUniform(self.weight, a=math.sqrt(5.0))

    def forward(self, x_s):
        return _ColumnParallelFn.apply(x_s, self.weight, self.bias, self.comm)


class RowParallelLinear(nn.Module):
    """Linear layer whose input features are split over the tensor-parallel group.

    Input: ``[M, in/tp]``.  Output: token shard ``[M/tp, out]`` (+ bias, + residual shard).
    """

    kType = "RowParallelLinear"

    def __init__(self, in_features: int, out_features: int, comm: TPComm, bias: bool = True, device=None,
                 dtype=torch.float32, in_local: Optional[int] = None):
        super().__init__()
        assert in_local is not None or in_features % comm.world == 0
        self.comm, self.in_features, self.out_features = comm, in_features, out_features
        self.in_local = in_local if in_local is not None else in_features // comm.world
        self.weight = torch.nn.Parameter(torch.empty(out_features, self.in_local, device=device, dtype=dtype))
        self.bias = _mark_sp(torch.nn.Parameter(torch.zeros(out_features, device=device, dtype=dtype))) if bias else None
        init.KaimingUniform(self.weight, a=math.sqrt(5.0))

    def forward(self, y, residual_s=None):
        return _RowParallelFn.apply(y, self.weight, self.bias, residual_s, self.comm)


class _VocabParallelEmbeddingPushFn(torch.autograd.Function):
    """The same result from the peer-memory kernels: each row is stored once, by the rank that holds it, into the
    token owner's shard; the backward pulls only the gradient rows a rank holds.  No reduction, 1 / world of the
    NVLink traffic of the masked gather + reduce-scatter below."""

    @staticmethod
    def forward(ctx, idx, w, comm: TPComm):
        idx = idx.contiguous()
        ctx.save_for_backward(idx)
        ctx.w, ctx.comm = w, comm
        return comm._fused.embedding_push(idx, w, w.shape[0] * comm.world)

    @staticmethod
    def backward(ctx, dx_s):
        (idx,) = ctx.saved_tensors
        w, comm = ctx.w, ctx.comm
        mg, acc = F_._grad_target(w)
        if mg is not None:
            if not acc:
                mg.zero_()
            comm._fused.embedding_pull_bwd(idx, dx_s.contiguous(), mg.view(w.shape))
            F_._grad_done(w)
            return None, None, None
        g = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        comm._fused.embedding_pull_bwd(idx, dx_s.contiguous(), g)
        return None, g.to(w.dtype), None


class _VocabParallelEmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, w, comm: TPComm):
        V = w.shape[0]
        lo = comm.rank * V
        local = idx - lo
        mask = (local < 0) | (local >= V)
        local = local.clamp(0, V - 1)
        out = torch.nn.functional.embedding(local, w)
        out = out.masked_fill(mask.unsqueeze(-1), 0.0)
        ctx.save_for_backward(local, mask)
        ctx.w, ctx.comm = w, comm
        M = out.numel() // out.shape[-1]
        return comm.reduce_scatter_rows(out.reshape(M, -1))

    @staticmethod
    def backward(ctx, dx_s):
        local, mask = ctx.saved_tensors
        w, comm = ctx.w, ctx.comm
        d = comm.all_gather_rows(dx_s.contiguous())
        d = d.masked_fill(mask.reshape(-1, 1), 0.0)
        mg, acc = F_._grad_target(w)
        if mg is not None:
            if not acc:
                mg.zero_()
            mg.view(w.shape).index_add_(0, local.reshape(-1), d.float())
            F_._grad_done(w)
            return None, None, None
        g = torch.zeros(w.shape, device=w.device, dtype=torch.float32)
        g.index_add_(0, local.reshape(-1), d.float())
        return None, g.to(w.dtype), None


class VocabParallelEmbedding(nn.Module):
    """Embedding table split by rows (vocabulary) over the tensor-parallel group.
    ``forward(idx [B, T])`` returns the token shard ``[B*T/tp, C]``."""

    kType = "VocabParallelEmbedding"

    def __init__(self, num_embeddings: int, embedding_dim: int, comm: TPComm, device=None, dtype=torch.float32):
        super().__init__()
        assert num_embeddings % comm.world == 0
        self.comm = comm
        self.num_local = num_embeddings // comm.world
        self.weight = torch.nn.Parameter(torch.empty(self.num_local, embedding_dim, device=device, dtype=dtype))
        init.Normal(self.weight, 0.0, 1.0)

    def forward(self, idx):
        w, comm = self.weight, self.comm
        vn = 8 if w.dtype == _bf16 else 4
        if (comm._fused is not None and w.is_cuda and w.dtype in (_bf16, torch.float32) and comm.world <= 16
                and idx.numel() % comm.world == 0 and w.shape[1] % vn == 0 and not F_.DETERMINISTIC_EMBEDDING_GRAD):
            return _VocabParallelEmbeddingPushFn.apply(idx, w, comm)
        return _VocabParallelEmbeddingFn.apply(idx, w, comm)


class _VocabParallelLossFn(torch.autograd.Function):
    """Mean cross entropy over vocabulary-sharded logits.

    Each rank computes its logits slice ``X W_r^T`` (X gathered from token shards), the ranks
    exchange per-row (max, sum-exp, target-logit) and every rank turns its slice into the
    gradient in place.  The full [M, V] logits never exist on one GPU.
    """

    @staticmethod
    def forward(ctx, x_s, w, targets, vocab_size, comm: TPComm):
        logits, X = comm.ag_gemm(x_s, w)
        M, Vl = logits.shape
        lo = comm.rank * Vl
        if logits.is_cuda and logits.dtype in (torch.float32, _bf16) and comm.world <= 16:
            # own kernels: one pass for the slice statistics, exchange of [M, 3] triples, one in-place gradient pass
            tgt = targets.reshape(-1).contiguous()
            table, dst, slot = comm.vp_stats_table(M, logits.device)
            C.xent_vp_stats(logits, tgt, dst, slot, lo, vocab_size)
            table = comm.vp_stats_publish(table, M)
            losses = C.xent_vp_grad(logits, tgt, table, lo, vocab_size, 1.0 / M)
            ctx.save_for_backward(X, w, logits)
            ctx.comm = comm
            return losses.mean()
        # CPU ranks (and groups beyond 16 ranks): the same exchange written with torch ops and three all-reduces
        lf = logits.float()
        col = torch.arange(Vl, device=logits.device) + lo
        lf = lf.masked_fill((col >= vocab_size).unsqueeze(0), float("-inf"))
        gmax = lf.max(dim=1).values
        comm.all_reduce(gmax, op=dist.ReduceOp.MAX)
        ex = torch.exp(lf - gmax.unsqueeze(1))
        ssum = ex.sum(dim=1)
        comm.all_reduce(ssum)
        tloc = targets.reshape(-1) - lo
        inr = (tloc >= 0) & (tloc < Vl)
        tl = lf.gather(1, tloc.clamp(0, Vl - 1).unsqueeze(1)).squeeze(1)
        tl = torch.where(inr, tl, torch.zeros_like(tl))
        comm.all_reduce(tl)
        lse = gmax + torch.log(ssum)
        loss = (lse - tl).mean()
        probs = ex / ssum.unsqueeze(1)
        probs[torch.arange(M, device=logits.device)[inr], tloc[inr]] -= 1.0
        dlogits = (probs / M).to(logits.dtype)
        ctx.save_for_backward(X, w, dlogits)
        ctx.comm = comm
        return loss

    @staticmethod
    def backward(ctx, dloss):
        X, w, dlogits = ctx.saved_tensors
        comm = ctx.comm
        dl = (dlogits.float() * dloss.float()).to(dlogits.dtype)
        dx_s = comm.gemm_rs(dl, w, b_mn=True)
        dw = _wgrad_any(dl, X, w)
        return dx_s, dw, None, None, None


def vocab_parallel_lm_head_loss(x_s, weight_local, targets, vocab_size: int, comm: TPComm):
    """Fused output projection + cross entropy with the vocabulary split over the group."""
    return _VocabParallelLossFn.apply(x_s, weight_local, targets, vocab_size, comm)
