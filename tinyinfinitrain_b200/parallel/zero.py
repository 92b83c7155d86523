"""Data parallelism with a ZeRO-1 distributed optimizer.

Every rank holds the full bf16 parameters and a full fp32 main-gradient buffer (written in
place by the wgrad kernels); optimizer state (fp32 master weights, Adam moments) is sharded:
rank r owns elements ``[r*S, (r+1)*S)`` of the flat parameter space.

``comm="fused"`` (default on GPUs): gradient and parameter buffers live in symmetric memory and
one kernel per bucket does reduce-scatter + scale + Adam + parameter all-gather over NVLink
(``csrc/kernels/comm.cu: rs_adam_ag_kernel``).  The flat space is cut into ``num_buckets``
contiguous buckets on parameter boundaries, each sharded over the ranks; as soon as backward has
produced every gradient of a bucket (the wgrad kernels report it through ``_on_grad_ready``) its
barrier + fused kernel are enqueued on a side stream, so the NVLink traffic and the optimizer math
of the deep layers run underneath the backward pass of the shallow ones.  The bucket holding the
tied embedding (written twice) and anything not reported are handled in ``step()``.  The default
is one bucket reduced in ``step()``; ``num_buckets > 1`` with ``overlap=True`` turns the overlap on.
``comm="nccl"``: the unfused baseline -- ``reduce_scatter_tensor``, local fused Adam,
``all_gather_into_tensor``.  On CPU (gloo) the same sharding logic runs with torch ops, which is
what the CPU multi-process tests exercise.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..optim.optimizers import FlatParams


class DistributedOptimizer:
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 group: Optional[dist.ProcessGroup] = None, comm: str = "fused", average: bool = True,
                 num_buckets: int = 1, overlap: bool = False, max_grad_norm: float = 0.0, mp_group=None, tp_world: int = 1):
        plist = [p for p in params]
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        dev, dt = plist[0].device, plist[0].dtype
        self.is_cuda = dev.type == "cuda"
        self.comm = comm if self.is_cuda else "torch"
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.t = 0
        self.grad_scale = (1.0 / self.world) if average else 1.0
        # > 0: clip the global L2 norm of the (averaged) gradient.  The norm needs the reduced gradient before the update
        # uses it, so the fused path reads its shard of the peers' gradients once more for the norm and every rank scales
        # its local buffer by the agreed coefficient before the fused reduce-scatter + Adam kernel runs.
        self.max_grad_norm = max_grad_norm
        self.mp_group, self.tp_world = mp_group, tp_world     # model-parallel layout for the global norm (see optim.clip_coefficient)
        if max_grad_norm > 0 and overlap:
            raise ValueError("gradient clipping needs the whole gradient before any bucket is updated: use overlap=False")
        align = 8 * self.world * 16
        # size the flat space first, then allocate (symmetric) buffers and bind the parameters to them
        total = self._flat_size(plist, align)
        self.gbuf = self.pbuf = None
        if self.comm == "fused":
            from .symm import DeviceBarrier, SymmetricBuffer

            self.gbuf = SymmetricBuffer(total, torch.float32, dev, self.group)
            self.pbuf = SymmetricBuffer(total, dt, dev, self.group)
            self.gbuf.tensor.zero_()
            self.pbuf.tensor.zero_()
            self.flat = FlatParams(plist, align_total=align, grad_buffer=self.gbuf.tensor, param_buffer=self.pbuf.tensor)
            self.barrier = DeviceBarrier(self.gbuf, channel=0)
        else:
            self.flat = FlatParams(plist, align_total=align)
        f = self.flat
        assert f.total == total and total % self.world == 0
        self.shard_n = total // self.world
        self.shard_off = self.rank * self.shard_n
        self.overlap = overlap and self.comm == "fused"
        self.side_blocks = 64  # CTAs of a bucket kernel that runs beside backward (leaves SMs to the GEMMs)
        self._plan_buckets(num_buckets if self.comm == "fused" else 1)
        # all ranks must start from identical parameters: broadcast rank 0's flat buffer
        dist.broadcast(f.param, src=dist.get_global_rank(self.group, 0) if self.group is not dist.group.WORLD else 0,
                       group=self.group)
        self.mixed = f.dtype != torch.float32
        if self.comm == "fused":
            # local state = this rank's slice of every bucket, concatenated
            pieces = [f.param[b["start"] + self.rank * b["shard"]: b["start"] + (self.rank + 1) * b["shard"]]
                      for b in self.buckets]
            self.master = torch.cat([x.float() for x in pieces]).contiguous()
        else:
            sl = slice(self.shard_off, self.shard_off + self.shard_n)
            self.master = f.param[sl].float().clone()
        self.m = torch.zeros(self.shard_n, device=dev, dtype=torch.float32)
        self.v = torch.zeros(self.shard_n, device=dev, dtype=torch.float32)
        self.dev_state = torch.tensor([0.0, 0.0, 0.0, lr], device=dev, dtype=torch.float32) if self.is_cuda else None
        self._gshard = torch.empty(self.shard_n, device=dev, dtype=torch.float32) if self.comm != "fused" else None
        self.clip_state = torch.tensor([0.0, 1.0], device=dev, dtype=torch.float32)     # {norm, coefficient}
        self._norm_buf = None
        if self.comm == "fused" and max_grad_norm > 0:
            from .symm import SymmetricBuffer

            self._norm_buf = SymmetricBuffer(64, torch.float32, dev, self.group)   # slot 0: this rank's squared shard norm
            self._norm_all = torch.zeros(1, device=dev, dtype=torch.float32)
        if self.is_cuda:
            torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)

    # ---- buckets -----------------------------------------------------------------------------------
    def _plan_buckets(self, nb: int) -> None:
        """Cuts [0, total) into up to ``nb`` buckets on parameter boundaries (offsets are multiples of
        128 elements, so every bucket divides evenly over up to 16 ranks in 8-element units)."""
        f = self.flat
        target = max(1, f.total // max(1, nb))
        bounds = [0]
        for p, off in zip(f.params, f.offsets):
            if off - bounds[-1] >= target and len(bounds) < nb:
                bounds.append(off)
        bounds.append(f.total)
        self.buckets = []
        local = 0
        for i in range(len(bounds) - 1):
            s, e = bounds[i], bounds[i + 1]
            shard = (e - s) // self.world
            self.buckets.append({"start": s, "end": e, "shard": shard, "local": local, "params": [], "pending": 0,
                                 "launched": False, "late": False})
            local += shard
        for p, off in zip(f.params, f.offsets):
            for b in self.buckets:
                if b["start"] <= off < b["end"]:
                    b["params"].append(p)
                    p._bucket = b
                    break
        self.comm_stream = None  # created at the first side-stream launch
        if self.overlap:
            for p in f.params:
                p._on_grad_ready = self._grad_ready
                p._expected = None  # reports per step, learned from the first step
        self._learned = False

    def _reset_pending(self) -> None:
        for b in self.buckets:
            b["pending"] = sum(p._expected for p in b["params"]) if self._learned else -1
            b["launched"] = False
        for p in self.flat.params:
            p._reports = 0
        self._ticked = False

    def _grad_ready(self, p) -> None:
        """Called by the kernel wrappers right after the launch that wrote ``p.main_grad``.  The first
        step only counts reports per parameter (a tied embedding reports twice, gradient accumulation
        multiplies every count); later steps launch a bucket when its last expected report arrives."""
        p._reports += 1
        if not self._learned:
            return
        b = p._bucket
        b["pending"] -= 1
        if b["pending"] == 0 and not b["late"] and not b["launched"]:
            self._launch_bucket(b, side=True)

    def _finish_learning(self) -> None:
        for p in self.flat.params:
            p._expected = p._reports
        for b in self.buckets:
            # a parameter that never reports (gradient through plain autograd) keeps its bucket for step()
            b["late"] = any(p._expected == 0 for p in b["params"])
        self._learned = True

    def _launch_bucket(self, b, side: bool) -> None:
        from .._lib import C

        b1, b2 = self.betas
        main = torch.cuda.current_stream(self.flat.device)
        if side and self.overlap and self.comm_stream is None:
            self.comm_stream = torch.cuda.Stream(device=self.flat.device)
        stream = self.comm_stream if (side and self.overlap) else main
        if stream is not main:
            stream.wait_stream(main)
        with torch.cuda.stream(stream):
            if not self._ticked:
                C.adam_tick(self.dev_state, b1, b2)
                self._ticked = True
            self.barrier()  # every rank has written this bucket's gradients
            lo, n = b["local"], b["shard"]
            C.rs_adam_ag(self.gbuf.ptrs, self.pbuf.ptrs, self.gbuf.mc_ptr, self.pbuf.mc_ptr, self.master[lo:lo + n],
                         self.m[lo:lo + n], self.v[lo:lo + n], b["start"] + self.rank * n, self.rank, self.lr, b1, b2,
                         self.eps, self.weight_decay, self.t + 1, self.grad_scale, self.dev_state,
                         self.side_blocks if stream is not main else 0)
        b["launched"] = True

    @staticmethod
    def _flat_size(plist, align: int) -> int:
        seen, off = set(), 0
        for p in plist:
            if id(p) in seen or not p.requires_grad:
                continue
            seen.add(id(p))
            off += (p.numel() + 127) // 128 * 128
        return (off + align - 1) // align * align

    @property
    def params(self):
        return self.flat.params

    def set_lr(self, lr: float) -> None:
        self.lr = lr
        if self.dev_state is not None:
            self.dev_state[3:4].fill_(lr)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flat.mark_fresh()
        if self.comm == "fused":
            self._reset_pending()

    ZeroGrad = zero_grad

    @torch.no_grad()
    def step(self) -> None:
        from .._lib import C

        f = self.flat
        f.finish_unwritten()
        self.t += 1
        b1, b2 = self.betas
        if self.comm == "fused":
            self.t -= 1  # buckets launched during backward used t + 1 already
            if not hasattr(self, "_ticked"):
                self._reset_pending()
            main = torch.cuda.current_stream(f.device)
            if self.max_grad_norm > 0:
                self._clip_fused()
            for b in self.buckets:
                if not b["launched"]:
                    # same stream as the early buckets: the barrier channel is used by one stream at a time
                    self._launch_bucket(b, side=True)
            if self.overlap:
                if self.comm_stream is not None:
                    main.wait_stream(self.comm_stream)
                if not self._learned:
                    self._finish_learning()
            self.t += 1
            self.barrier()  # every shard of the new parameters has landed everywhere; gradients may be reused
            self._reset_pending()
            return
        dist.reduce_scatter_tensor(self._gshard, f.grad, op=dist.ReduceOp.SUM, group=self.group) \
            if self.is_cuda else self._cpu_reduce_scatter()
        if self.max_grad_norm > 0:
            self._clip_shard()
        sl = slice(self.shard_off, self.shard_off + self.shard_n)
        if self.is_cuda:
            C.adam_tick(self.dev_state, b1, b2)
            C.adam_flat(self.master, f.param[sl] if self.mixed else None, self._gshard, self.m, self.v, self.lr, b1,
                        b2, self.eps, self.weight_decay, self.t, self.grad_scale, self.dev_state)
            if not self.mixed:
                f.param[sl].copy_(self.master)
            dist.all_gather_into_tensor(f.param, f.param[sl].clone(), group=self.group)
        else:
            g = self._gshard * self.grad_scale
            self.m.mul_(b1).add_(g, alpha=1 - b1)
            self.v.mul_(b2).addcmul_(g, g, value=1 - b2)
            mh, vh = self.m / (1 - b1 ** self.t), self.v / (1 - b2 ** self.t)
            self.master.sub_(self.lr * (mh / (vh.sqrt() + self.eps) + self.weight_decay * self.master))
            shards = [torch.empty(self.shard_n, dtype=f.dtype) for _ in range(self.world)]
            dist.all_gather(shards, self.master.to(f.dtype), group=self.group)
            f.param.copy_(torch.cat(shards))

    Step = step

    def _clip_fused(self) -> None:
        """Global-norm clipping on the fused path: barrier (all gradients written) -> squared norm of this rank's shard
        of the summed gradient (NVLink read), separately for the region of tensor-parallel-replicated parameters ->
        exchange of the ranks' partial results through symmetric memory -> coefficient -> every rank scales its own
        gradient buffer.  The regular bucket launch that follows starts with its own barrier, which also orders the
        scaling before the peers' reads."""
        from .._lib import C
        from ..optim.optimizers import clip_coefficient

        n_rep = self.flat.n_replicated
        self.barrier()
        k = 0                                                # slots alternate: whole shard, its replicated part
        self._norm_buf.tensor[:2 * len(self.buckets)].zero_()
        for b in self.buckets:
            lo = b["start"] + self.rank * b["shard"]
            hi = lo + b["shard"]
            C.rs_grad_sumsq(self.gbuf.ptrs, self.gbuf.mc_ptr, lo, b["shard"], self.rank, self._norm_buf.tensor[k:k + 1])
            k += 1
            rep_hi = min(hi, n_rep)
            if rep_hi > lo:                                  # part of this shard lies in the replicated region
                C.rs_grad_sumsq(self.gbuf.ptrs, self.gbuf.mc_ptr, lo, rep_hi - lo, self.rank, self._norm_buf.tensor[k:k + 1])
            k += 1
        self.barrier()
        sums = torch.empty(k, device=self.flat.device, dtype=torch.float32)
        C.allreduce_small(self._norm_buf.ptrs, sums, 0)       # sum over the data-parallel ranks, slot by slot
        total = sums[0::2].sum()
        rep = sums[1::2].sum()
        coef = clip_coefficient(total, rep, self.tp_world, self.mp_group, self.grad_scale, self.max_grad_norm, self.clip_state)
        C.scale_by_dev_(self.gbuf.tensor, coef)

    def _clip_shard(self) -> None:
        """Unfused path: squared norm of the reduced shard (and of its part in the replicated region), summed over the
        data-parallel ranks, then the shard is scaled."""
        from ..optim.optimizers import clip_coefficient

        n_rep = self.flat.n_replicated
        g = self._gshard.float()
        rep_n = max(0, min(self.shard_off + self.shard_n, n_rep) - self.shard_off)
        sq = torch.stack([(g ** 2).sum(), (g[:rep_n] ** 2).sum()])
        dist.all_reduce(sq, group=self.group)
        coef = clip_coefficient(sq[0], sq[1], self.tp_world, self.mp_group, self.grad_scale, self.max_grad_norm, self.clip_state)
        self._gshard.mul_(coef)

    def grad_norm(self) -> float:
        return float(self.clip_state[0])

    def _cpu_reduce_scatter(self) -> None:
        # gloo has no reduce_scatter: all-reduce then slice (CPU logic tests only)
        g = self.flat.grad.clone()
        dist.all_reduce(g, group=self.group)
        self._gshard.copy_(g[self.shard_off:self.shard_off + self.shard_n])

    # ---- sharded checkpoint state ------------------------------------------------------------
    def state_dict(self):
        return {"t": self.t, "rank": self.rank, "world": self.world, "shard_off": self.shard_off,
                "layout": [(b["start"], b["shard"]) for b in self.buckets] if self.comm == "fused" else [(0, self.shard_n)],
                "master": self.master.cpu(), "m": self.m.cpu(), "v": self.v.cpu()}

    def load_state_dict(self, sd) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank, "optimizer shard belongs to another layout"
        mine = [(b["start"], b["shard"]) for b in self.buckets] if self.comm == "fused" else [(0, self.shard_n)]
        assert [tuple(x) for x in sd.get("layout", mine)] == mine, "checkpoint was written with another bucket layout"
        self.t = int(sd["t"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if self.dev_state is not None:
            b1, b2 = self.betas
            self.dev_state[0] = float(self.t)
            self.dev_state[1] = 1.0 - b1 ** self.t if self.t else 0.0
            self.dev_state[2] = 1.0 - b2 ** self.t if self.t else 0.0
        self._gather_params_from_master()

    def _gather_params_from_master(self) -> None:
        """Rebuilds the full parameter buffer of every rank from the ranks' master-weight shards (after a resume: a
        rank only restored its own shard).  One all-gather per bucket on the process group; not on the step path."""
        f = self.flat
        lo = 0
        for b in (self.buckets if self.comm == "fused" else [{"start": 0, "shard": self.shard_n}]):
            n = b["shard"]
            mine = self.master[lo:lo + n].to(f.dtype).contiguous()
            parts = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(parts, mine, group=self.group)
            f.param[b["start"]:b["start"] + n * self.world].copy_(torch.cat(parts))
            lo += n
        if self.is_cuda:
            torch.cuda.synchronize(f.device)
        dist.barrier(group=self.group)

class AllReduceOptimizer:
    """Plain data parallelism (``--zero_stage 0``): the flat fp32 gradient buffer is all-reduced over the group
    (one NCCL / gloo collective on the whole buffer) and every rank runs the full Adam update on identical averaged
    gradients.  It keeps full optimizer state on every rank and exists as the unsharded baseline next to
    :class:`DistributedOptimizer`, whose fused kernel is the product."""

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 group: Optional[dist.ProcessGroup] = None, max_grad_norm: float = 0.0, mp_group=None, tp_world: int = 1,
                 comm: str = "nccl"):
        """``comm="symm"``: the gradient buffer is allocated in symmetric memory and summed by this package's own
        two-shot all-reduce kernel (multimem through NVSwitch, or peer loads) instead of NCCL."""
        from ..optim.optimizers import FlatParams, MixedPrecisionAdam

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        plist = [p for p in params]
        self.coll = None
        flat = plist
        if comm == "symm" and plist and plist[0].is_cuda:
            from .collectives import SymmCollective

            align = 128 * self.world
            total = DistributedOptimizer._flat_size(plist, align)
            self.coll = SymmCollective(total, torch.float32, plist[0].device, self.group, channel=0)
            flat = FlatParams(plist, align_total=align, grad_buffer=self.coll.tensor)
        self.inner = MixedPrecisionAdam(flat, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                                        grad_scale=1.0 / self.world, max_grad_norm=max_grad_norm,
                                        mp_group=mp_group,
                                        tp_world=tp_world)
        self.flat = self.inner.flat
        src = dist.get_global_rank(self.group, 0) if self.group is not dist.group.WORLD else 0
        dist.broadcast(self.flat.param, src=src, group=self.group)       # all replicas start from rank 0's weights
        if self.inner.mixed:
            self.inner.master.copy_(self.flat.param.float())

    @property
    def params(self):
        return self.inner.params

    def set_lr(self, lr: float) -> None:
        self.inner.set_lr(lr)

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.inner.zero_grad()

    ZeroGrad = zero_grad

    @torch.no_grad()
    def step(self) -> None:
        self.flat.finish_unwritten()
        if self.coll is not None:
            self.coll.all_reduce_()                                       # own kernel, in place on the symmetric buffer
        else:
            dist.all_reduce(self.flat.grad, group=self.group)             # sum; the Adam kernel applies 1 / world
        self.inner.step()

    Step = step

    def grad_norm(self) -> float:
        return self.inner.grad_norm()

    def state_dict(self):
        return self.inner.state_dict()

    def load_state_dict(self, sd) -> None:
        self.inner.load_state_dict(sd)
