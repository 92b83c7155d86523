"""Data parallelism with a ZeRO-1 distributed optimizer.

Every rank holds the full bf16 parameters and a full fp32 main-gradient buffer (written in
place by the wgrad kernels); optimizer state (fp32 master weights, Adam moments) is sharded:
rank r owns elements ``[r*S, (r+1)*S)`` of the flat parameter space.

``comm="fused"`` (default on GPUs): gradient and parameter buffers live in symmetric memory and
one kernel per step does reduce-scatter + scale + Adam + parameter all-gather over NVLink
(``csrc/kernels/comm.cu: rs_adam_ag_kernel``), bracketed by two device-side barriers.
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
                 group: Optional[dist.ProcessGroup] = None, comm: str = "fused", average: bool = True):
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
        # all ranks must start from identical parameters: broadcast rank 0's flat buffer
        dist.broadcast(f.param, src=dist.get_global_rank(self.group, 0) if self.group is not dist.group.WORLD else 0,
                       group=self.group)
        sl = slice(self.shard_off, self.shard_off + self.shard_n)
        self.mixed = f.dtype != torch.float32
        self.master = f.param[sl].float().clone()
        self.m = torch.zeros(self.shard_n, device=dev, dtype=torch.float32)
        self.v = torch.zeros(self.shard_n, device=dev, dtype=torch.float32)
        self.dev_state = torch.tensor([0.0, 0.0, 0.0, lr], device=dev, dtype=torch.float32) if self.is_cuda else None
        self._gshard = torch.empty(self.shard_n, device=dev, dtype=torch.float32) if self.comm != "fused" else None
        if self.is_cuda:
            torch.cuda.synchronize(dev)
        dist.barrier(group=self.group)

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

    ZeroGrad = zero_grad

    @torch.no_grad()
    def step(self) -> None:
        from .._lib import C

        f = self.flat
        f.finish_unwritten()
        self.t += 1
        b1, b2 = self.betas
        if self.comm == "fused":
            C.adam_tick(self.dev_state, b1, b2)
            self.barrier()  # every rank has finished writing its gradients (and reading its parameters)
            C.rs_adam_ag(self.gbuf.ptrs, self.pbuf.ptrs, self.gbuf.mc_ptr, self.pbuf.mc_ptr, self.master, self.m,
                         self.v, self.shard_off, self.rank, self.lr, b1, b2, self.eps, self.weight_decay, self.t,
                         self.grad_scale, self.dev_state)
            self.barrier()  # every shard of the new parameters has landed everywhere; gradients may be reused
            return
        dist.reduce_scatter_tensor(self._gshard, f.grad, op=dist.ReduceOp.SUM, group=self.group) \
            if self.is_cuda else self._cpu_reduce_scatter()
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

    def _cpu_reduce_scatter(self) -> None:
        # gloo has no reduce_scatter: all-reduce then slice (CPU logic tests only)
        g = self.flat.grad.clone()
        dist.all_reduce(g, group=self.group)
        self._gshard.copy_(g[self.shard_off:self.shard_off + self.shard_n])

    # ---- sharded checkpoint state ------------------------------------------------------------
    def state_dict(self):
        return {"t": self.t, "rank": self.rank, "world": self.world, "shard_off": self.shard_off,
                "master": self.master.cpu(), "m": self.m.cpu(), "v": self.v.cpu()}

    def load_state_dict(self, sd) -> None:
        assert sd["world"] == self.world and sd["rank"] == self.rank, "optimizer shard belongs to another layout"
        self.t = int(sd["t"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if self.dev_state is not None:
            b1, b2 = self.betas
            self.dev_state[0] = float(self.t)
            self.dev_state[1] = 1.0 - b1 ** self.t if self.t else 0.0
            self.dev_state[2] = 1.0 - b2 ** self.t if self.t else 0.0
