"""SGD and Adam with the reference's API, plus flat mixed-precision Adam.

Reference: infini_train/include/optimizer.h:9-47, src/optimizer.cc:10-53.  The
expected Adam math is the closed form of test/optimizer/test_adam.cc:50-58:
``m = b1 m + (1-b1) g; v = b2 v + (1-b2) g^2; p -= lr (m/(1-b1^t)) / (sqrt(v/(1-b2^t)) + eps)``.
``weight_decay`` (decoupled, AdamW) is an addition; 0 reproduces the reference.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch

from .._lib import C


class Optimizer:
    def __init__(self, params: Iterable[torch.Tensor]):
        seen, self.params = set(), []
        for p in params:  # tied tensors are updated once
            if id(p) not in seen:
                seen.add(id(p))
                self.params.append(p)

    def ZeroGrad(self) -> None:
        for p in self.params:
            if p.grad is not None:
                p.grad.zero_()

    def Step(self) -> None:
        raise NotImplementedError

    # pythonic aliases
    def zero_grad(self, set_to_none: bool = False) -> None:
        if set_to_none:
            for p in self.params:
                p.grad = None
        else:
            self.ZeroGrad()

    def step(self) -> None:
        self.Step()


class SGD(Optimizer):
    """p -= lr * grad (no momentum, no weight decay: optimizer.cc:18-27)."""

    def __init__(self, params, learning_rate: float):
        super().__init__(params)
        self.lr = learning_rate

    @torch.no_grad()
    def Step(self) -> None:
        for p in self.params:
            if p.grad is None:
                continue
            if p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32 and p.is_contiguous():
                C.sgd_flat(p.data.view(-1), None, p.grad.contiguous().view(-1), self.lr)
            else:
                p.add_(p.grad.to(p.dtype), alpha=-self.lr)


class Adam(Optimizer):
    """Bias-corrected Adam; per-parameter fp32 moments (and fp32 master copies of bf16 parameters)."""

    def __init__(self, params, learning_rate: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999,
                 eps: float = 1e-8, weight_decay: float = 0.0):
        super().__init__(params)
        self.lr, self.beta1, self.beta2, self.eps, self.weight_decay = learning_rate, beta1, beta2, eps, weight_decay
        self.t = 0
        self.m = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.v = [torch.zeros_like(p, dtype=torch.float32) for p in self.params]
        self.master: List[Optional[torch.Tensor]] = [
            p.detach().float().clone() if p.dtype != torch.float32 else None for p in self.params]

    @torch.no_grad()
    def Step(self) -> None:
        self.t += 1
        t = self.t
        for i, p in enumerate(self.params):
            if p.grad is None:
                continue
            m, v, master = self.m[i], self.v[i], self.master[i]
            g = p.grad
            if p.is_cuda and p.is_contiguous():
                g32 = g.contiguous().view(-1) if g.dtype == torch.float32 else g.float().contiguous().view(-1)
                if master is None:
                    C.adam_flat(p.data.view(-1), None, g32, m.view(-1), v.view(-1), self.lr, self.beta1, self.beta2,
                                self.eps, self.weight_decay, t, 1.0)
                else:
                    C.adam_flat(master.view(-1), p.data.view(-1), g32, m.view(-1), v.view(-1), self.lr, self.beta1,
                                self.beta2, self.eps, self.weight_decay, t, 1.0)
                continue
            g32 = g.float()
            m.mul_(self.beta1).add_(g32, alpha=1.0 - self.beta1)
            v.mul_(self.beta2).addcmul_(g32, g32, value=1.0 - self.beta2)
            mh = m / (1.0 - self.beta1 ** t)
            vh = v / (1.0 - self.beta2 ** t)
            w = master if master is not None else p
            w.sub_(self.lr * (mh / (vh.sqrt() + self.eps) + self.weight_decay * w))
            if master is not None:
                p.copy_(master.to(p.dtype))


def _round_up(n: int, m: int) -> int:
    return (n + m - 1) // m * m


class FlatParams:
    """Lays the parameters of a model out in flat buffers.

    * ``param``  -- the compute copy (bf16 or fp32); every ``p.data`` becomes a view of it,
    * ``grad``   -- fp32 main gradients; ``p.main_grad`` views it and the wgrad kernels
      accumulate there directly,
    * ``master`` -- fp32 master weights (aliases ``param`` when the model is fp32).

    Offsets are padded to 128 elements so each view is 16-byte aligned for TMA and
    128-bit accesses, and ``total`` is padded to ``align_total`` elements so it can be
    split evenly across data-parallel ranks.
    """

    def __init__(self, params: Iterable[torch.nn.Parameter], align_total: int = 128, grad_buffer=None,
                 param_buffer=None):
        seen, plist = set(), []
        for p in params:
            if id(p) not in seen and p.requires_grad:
                seen.add(id(p))
                plist.append(p)
        assert plist, "no trainable parameters"
        # parameters that are replicated over a tensor-parallel group (flagged ``_sp_grad_sync`` by parallel.tp) go first,
        # in their original order: their gradients then form ONE contiguous region [0, n_replicated) that the group
        # all-reduces in a single collective and that the gradient norm counts once.  Models without such
        # parameters keep their order.
        plist = [p for p in plist if getattr(p, "_sp_grad_sync", False)] + \
                [p for p in plist if not getattr(p, "_sp_grad_sync", False)]
        self.params = plist
        dev, dt = plist[0].device, plist[0].dtype
        assert all(p.device == dev and p.dtype == dt for p in plist), "parameters must share device and dtype"
        self.offsets, off = [], 0
        for p in plist:
            self.offsets.append(off)
            off += _round_up(p.numel(), 128)
        self.total = _round_up(off, align_total)
        self.n_replicated = 0
        for p, o in zip(plist, self.offsets):
            if getattr(p, "_sp_grad_sync", False):
                self.n_replicated = o + _round_up(p.numel(), 128)
        self.device, self.dtype = dev, dt
        self.param = param_buffer if param_buffer is not None else torch.zeros(self.total, device=dev, dtype=dt)
        self.grad = grad_buffer if grad_buffer is not None else torch.zeros(self.total, device=dev,
                                                                            dtype=torch.float32)
        assert self.param.numel() >= self.total and self.grad.numel() >= self.total
        with torch.no_grad():
            for p, o in zip(plist, self.offsets):
                n = p.numel()
                self.param[o:o + n].copy_(p.detach().reshape(-1))
                p.data = self.param[o:o + n].view(p.shape)
                p.main_grad = self.grad[o:o + n].view(p.shape)
                p._fresh_grad = True
                p._flat = self
                p.grad = None

    def mark_fresh(self) -> None:
        """Next gradient write of every parameter overwrites instead of accumulating."""
        for p in self.params:
            p._fresh_grad = True

    def finish_unwritten(self) -> None:
        """Folds gradients that arrived through plain autograd (``p.grad``: CPU tensors, fp32 ops,
        user-defined ops) into the main-gradient buffer, and zeroes parameters that got none."""
        for p in self.params:
            if p.grad is not None:
                if p._fresh_grad:
                    p.main_grad.copy_(p.grad)
                else:
                    p.main_grad.add_(p.grad)
                p._fresh_grad = False
                p.grad = None
            elif p._fresh_grad:
                p.main_grad.zero_()
                p._fresh_grad = False


def clip_coefficient(total_sq, replicated_sq, tp_world: int, mp_group, grad_scale: float, max_norm: float, clip_state):
    """Global gradient norm and clip coefficient from this rank's sums of squares.

    ``total_sq``: all local parameters; ``replicated_sq``: the part that belongs to parameters replicated over the
    tensor-parallel group (counted once in the global norm, so each of the ``tp_world`` copies contributes 1 / tp_world).
    ``mp_group``: the ranks that together hold one model replica (tensor x pipeline), or None.  Writes {norm, coefficient}
    into ``clip_state`` (device tensor of two floats) and returns the coefficient as a 1-element tensor view."""
    import torch.distributed as dist

    contrib = total_sq.reshape(1).clone()
    if tp_world > 1 and replicated_sq is not None:
        contrib -= (1.0 - 1.0 / tp_world) * replicated_sq.reshape(1)
    if mp_group is not None and dist.get_world_size(mp_group) > 1:
        dist.all_reduce(contrib, group=mp_group)
    norm = contrib.clamp_min(0).sqrt() * grad_scale
    clip_state[0:1].copy_(norm)
    clip_state[1:2].copy_(torch.clamp(max_norm / (norm + 1e-6), max=1.0))
    return clip_state[1:2]


class MixedPrecisionAdam:
    """Adam/AdamW over :class:`FlatParams`: one fused kernel launch per step.

    bf16 parameters keep fp32 master weights; the kernel reads the fp32 main gradient,
    updates master/m/v and writes the rounded bf16 parameters in the same pass
    (csrc/kernels/optim.cu).  fp32 models update the parameters in place.
    """

    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 grad_scale: float = 1.0, max_grad_norm: float = 0.0, mp_group=None, tp_world: int = 1):
        self.flat = params if isinstance(params, FlatParams) else FlatParams(params)
        # model-parallel layout for the global gradient norm: the group holding one model replica and the size of
        # its tensor-parallel dimension (parameters flagged as replicated there are counted once)
        self.mp_group, self.tp_world = mp_group, tp_world
        f = self.flat
        self.lr, self.betas, self.eps, self.weight_decay, self.grad_scale = lr, betas, eps, weight_decay, grad_scale
        # > 0: the global L2 norm of (grad_scale * gradient) is clipped to this value before the update; the norm and
        # the coefficient live in device memory (``clip_state``: {norm, coefficient}), so a captured step stays correct
        self.max_grad_norm = max_grad_norm
        self.clip_state = torch.tensor([0.0, 1.0], device=f.device, dtype=torch.float32)
        self.t = 0
        self.mixed = f.dtype != torch.float32
        self.master = f.param.float().clone() if self.mixed else f.param
        self.m = torch.zeros(f.total, device=f.device, dtype=torch.float32)
        self.v = torch.zeros(f.total, device=f.device, dtype=torch.float32)
        # {t, 1-b1^t, 1-b2^t, lr} on the device: the step counter advances inside the
        # captured work, so a CUDA graph of the step stays correct across replays.
        self.dev_state = (torch.tensor([0.0, 0.0, 0.0, lr], device=f.device, dtype=torch.float32)
                          if f.device.type == "cuda" else None)

    def set_lr(self, lr: float) -> None:
        self.lr = lr
        if self.dev_state is not None:
            self.dev_state[3:4].fill_(lr)

    @property
    def params(self):
        return self.flat.params

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.flat.mark_fresh()

    ZeroGrad = zero_grad

    @torch.no_grad()
    def step(self) -> None:
        f = self.flat
        f.finish_unwritten()
        self.t += 1
        b1, b2 = self.betas
        if f.device.type == "cuda":
            if self.max_grad_norm > 0 and self.mp_group is None:
                C.clip_grad_norm_(f.grad, self.max_grad_norm, self.grad_scale, self.clip_state)
            elif self.max_grad_norm > 0:
                sq = torch.zeros(2, device=f.device, dtype=torch.float32)
                C.sumsq_(f.grad, sq[0:1])
                C.sumsq_(f.grad[:f.n_replicated], sq[1:2])
                coef = clip_coefficient(sq[0], sq[1], self.tp_world, self.mp_group, self.grad_scale, self.max_grad_norm,
                                        self.clip_state)
                C.scale_by_dev_(f.grad, coef)
            C.adam_tick(self.dev_state, b1, b2)
            C.adam_flat(self.master, f.param if self.mixed else None, f.grad, self.m, self.v, self.lr, b1, b2,
                        self.eps, self.weight_decay, self.t, self.grad_scale, self.dev_state)
            return
        if self.max_grad_norm > 0:
            coef = clip_coefficient((f.grad ** 2).sum(), (f.grad[:f.n_replicated] ** 2).sum(), self.tp_world, self.mp_group,
                                    self.grad_scale, self.max_grad_norm, self.clip_state)
            f.grad.mul_(coef)
        g = f.grad * self.grad_scale
        self.m.mul_(b1).add_(g, alpha=1 - b1)
        self.v.mul_(b2).addcmul_(g, g, value=1 - b2)
        mh, vh = self.m / (1 - b1 ** self.t), self.v / (1 - b2 ** self.t)
        self.master.sub_(self.lr * (mh / (vh.sqrt() + self.eps) + self.weight_decay * self.master))
        if self.mixed:
            f.param.copy_(self.master.to(f.dtype))

    Step = step

    def grad_norm(self) -> float:
        """Norm of the last clipped step's gradient (before clipping); reads device memory, so it synchronises."""
        return float(self.clip_state[0])

    def state_dict(self):
        return {"t": self.t, "master": self.master, "m": self.m, "v": self.v}

    def load_state_dict(self, sd):
        self.t = int(sd["t"])
        self.master.copy_(sd["master"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if self.mixed:
            self.flat.param.copy_(self.master.to(self.flat.dtype))
        if self.dev_state is not None:
            b1, b2 = self.betas
            self.dev_state[0] = float(self.t)
            self.dev_state[1] = 1.0 - b1 ** self.t if self.t else 0.0
            self.dev_state[2] = 1.0 - b2 ** self.t if self.t else 0.0
