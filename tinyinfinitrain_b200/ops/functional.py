"""Autograd functions over the sm_100a kernels, with CPU reference paths.

Each public function takes torch tensors.  CUDA tensors run the hand-written
kernels of ``csrc/kernels`` (bf16 on tcgen05 tensor cores, fp32 on SIMT
kernels for API parity); CPU tensors run plain PyTorch fp32 math, which is the
numerical oracle the GPU tests compare against.

Weight gradients: a parameter that carries a ``main_grad`` attribute (an fp32
view into a flat gradient buffer owned by the optimizer / data-parallel
wrapper) gets its gradient accumulated there by the kernel, and autograd sees
``None`` for it.  ``param._fresh_grad = True`` means "overwrite instead of
accumulate" for the first write of a step, which replaces a zero-fill pass.
Parameters without ``main_grad`` get an ordinary ``.grad``.

Reference semantics: infini_train/src/kernels/cpu/*.cc (Linear :36-123 of
linear.cc, LayerNorm layernorm.cc:19-135, CrossEntropy cross_entropy.cc:17-96,
Embedding embedding.cc:9-54, Softmax softmax.cc:11-80).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn.functional as F

from .._lib import C

EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_DGELU, EPI_BIAS_RESIDUAL = 0, 1, 2, 3, 4
# TITB200_DETERMINISTIC=1: the token-embedding gradient is built by a sorted segment reduction instead of fp32 atomics
# (the one reduction of the training step whose summation order otherwise depends on timing)
DETERMINISTIC_EMBEDDING_GRAD = os.environ.get("TITB200_DETERMINISTIC", "0") == "1"

_bf16 = torch.bfloat16


# --------------------------------------------------------------------------- helpers
def _grad_target(p: torch.Tensor):
    """(buffer, accumulate) for writing p's gradient into its fp32 main_grad, or (None, False)."""
    mg = getattr(p, "main_grad", None)
    if mg is None:
        return None, False
    fresh = getattr(p, "_fresh_grad", False)
    if fresh:
        p._fresh_grad = False
    return mg, not fresh


def _grad_done(p: torch.Tensor):
    cb = getattr(p, "_on_grad_ready", None)
    if cb is not None:
        cb(p)


def _wgrad(dy2: torch.Tensor, x2: torch.Tensor, w: torch.Tensor, alpha=None):
    """dW[N, K] = dy2^T . x2 for dy2 [M, N], x2 [M, K] (both operands MN-major)."""
    mg, acc = _grad_target(w)
    if mg is not None:
        C.gemm(dy2, x2, True, True, out=mg.view(dy2.shape[1], x2.shape[1]), accumulate=acc, alpha=alpha)
        _grad_done(w)
        return None
    return C.gemm(dy2, x2, True, True, alpha=alpha)[0].view_as(w)


def _bgrad(dy2: torch.Tensor, b: torch.Tensor):
    mg, acc = _grad_target(b)
    if mg is not None:
        C.colsum(dy2, out=mg, accumulate=acc)
        _grad_done(b)
        return None
    return C.colsum(dy2).to(b.dtype)


def gelu_ref(x: torch.Tensor) -> torch.Tensor:
    """tanh-form GELU of example/gpt2/net.cc:46-51."""
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x * x * x)))


# ----------------------------------------------------------------------------- linear
class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ b) (+ residual) on tcgen05; dgrad and wgrad reuse the same kernel."""

    @staticmethod
    def forward(ctx, x, w, b, residual):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        N = w.shape[0]
        # the output is allocated in its final shape so that it is not a view (callers may modify it in place)
        y = torch.empty(*x.shape[:-1], N, device=x.device, dtype=x.dtype)
        y2 = y.view(-1, N)
        if residual is not None:
            C.gemm(x2, w, epilogue=EPI_BIAS_RESIDUAL, bias=b, aux_in=residual.reshape(-1, N), out=y2)
        elif b is not None:
            C.gemm(x2, w, epilogue=EPI_BIAS, bias=b, out=y2)
        else:
            C.gemm(x2, w, out=y2)
        ctx.save_for_backward(x2, w)
        ctx.b = b
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            dx = C.gemm(dy2, w, False, True)[0].view(ctx.xshape)
        dw = _wgrad(dy2, x2, w) if ctx.needs_input_grad[1] else None
        db = _bgrad(dy2, ctx.b) if (ctx.b is not None and ctx.needs_input_grad[2]) else None
        dres = dy if ctx.has_res else None
        return dx, dw, db, dres


class _LinearF32Fn(torch.autograd.Function):
    """fp32 tensors on the GPU: SIMT SGEMM (API parity with the reference's fp32 Linear)."""

    @staticmethod
    def forward(ctx, x, w, b):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        y = C.sgemm(x2, w.contiguous(), False, True)
        if b is not None:
            y = C.binary_fwd(0, y, b)
        ctx.save_for_backward(x2, w)
        ctx.has_b = b is not None
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        dx = C.sgemm(dy2, w.contiguous(), False, False).view(ctx.xshape)
        dw = C.sgemm(dy2, x2, True, False)
        db = C.colsum(dy2) if ctx.has_b else None
        return dx, dw, db


def linear(x, weight, bias=None, residual=None):
    """``x @ weight.T + bias (+ residual)`` with ``weight`` of shape [out, in]."""
    if not x.is_cuda:
        y = F.linear(x, weight, bias)
        return y + residual if residual is not None else y
    if x.dtype == _bf16:
        return _LinearFn.apply(x, weight, bias, residual)
    y = _LinearF32Fn.apply(x, weight, bias)
    return y + residual if residual is not None else y


class _MLPGeluFn(torch.autograd.Function):
    """GPT-2 MLP block: y = residual + gelu(x W1^T + b1) W2^T + b2.

    Forward: the first GEMM's epilogue writes both the pre-activation and the GELU
    output; the second adds bias and residual.  Backward: the dgrad GEMM through W2
    multiplies by gelu'(pre) in its epilogue, so no standalone activation kernel runs.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, residual):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        act, pre = C.gemm(x2, w1, epilogue=EPI_BIAS_GELU, bias=b1, want_aux_out=True)
        if residual is not None:
            y = C.gemm(act, w2, epilogue=EPI_BIAS_RESIDUAL, bias=b2, aux_in=residual.reshape(-1, w2.shape[0]))[0]
        else:
            y = C.gemm(act, w2, epilogue=EPI_BIAS, bias=b2)[0]
        ctx.save_for_backward(x2, w1, w2, pre, act)
        ctx.b1, ctx.b2 = b1, b2
        ctx.has_res = residual is not None
        ctx.xshape = x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w1, w2, pre, act = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dpre = C.gemm(dy2, w2, False, True, epilogue=EPI_DGELU, aux_in=pre)[0]
        dw2 = _wgrad(dy2, act, w2)
        db2 = _bgrad(dy2, ctx.b2) if ctx.b2 is not None else None
        dx = C.gemm(dpre, w1, False, True)[0].view(ctx.xshape)
        dw1 = _wgrad(dpre, x2, w1)
        db1 = _bgrad(dpre, ctx.b1) if ctx.b1 is not None else None
        return dx, dw1, db1, dw2, db2, (dy if ctx.has_res else None)


def mlp_gelu(x, w1, b1, w2, b2, residual=None):
    if x.is_cuda and x.dtype == _bf16:
        return _MLPGeluFn.apply(x, w1, b1, w2, b2, residual)
    h = gelu(linear(x, w1, b1))
    return linear(h, w2, b2, residual)


# ----------------------------------------------------------------------------- matmul
class _MatmulFn(torch.autograd.Function):
    """Batched [..., M, K] @ [..., K, N]; one tcgen05 launch per batch entry (bf16) or SGEMM (fp32)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        M, K, N = a.shape[-2], a.shape[-1], b.shape[-1]
        a3 = a.reshape(-1, M, K).contiguous()
        b3 = b.reshape(-1, K, N).contiguous()
        nb = a3.shape[0]
        assert b3.shape[0] == nb, "matmul: both operands must carry the same batch dims"
        out = torch.empty(nb, M, N, device=a.device, dtype=a.dtype)
        bf = a.dtype == _bf16 and K % 8 == 0 and N % 8 == 0
        for i in range(nb):
            if bf:
                C.gemm(a3[i], b3[i], False, True, out=out[i])
            else:
                af, bf_ = a3[i].float(), b3[i].float()
                out[i].copy_(C.sgemm(af, bf_, False, False))
        return out.view(*a.shape[:-2], M, N)

    @staticmethod
    def backward(ctx, dc):
        a, b = ctx.saved_tensors
        M, K, N = a.shape[-2], a.shape[-1], b.shape[-1]
        a3 = a.reshape(-1, M, K).contiguous()
        b3 = b.reshape(-1, K, N).contiguous()
        d3 = dc.reshape(-1, M, N).contiguous()
        da = torch.empty_like(a3)
        db = torch.empty_like(b3)
        bf = a.dtype == _bf16 and K % 8 == 0 and N % 8 == 0 and M % 8 == 0
        for i in range(a3.shape[0]):
            if bf:
                C.gemm(d3[i], b3[i], False, False, out=da[i])  # dA = dC B^T : B [K,N] is K-major for this product
                C.gemm(a3[i], d3[i], True, True, out=db[i])    # dB = A^T dC
            else:
                da[i].copy_(C.sgemm(d3[i].float(), b3[i].float(), False, True))
                db[i].copy_(C.sgemm(a3[i].float(), d3[i].float(), True, False))
        return da.view_as(a), db.view_as(b)


def matmul(a, b):
    if not a.is_cuda:
        return torch.matmul(a, b)
    return _MatmulFn.apply(a, b)


# ------------------------------------------------------------------------------ norms
class _LayerNormFn(torch.autograd.Function):
    """fork=True also returns x itself: the caller feeds that alias to the residual connection, and backward then
    receives the residual gradient as a second argument and adds it inside the norm kernel."""

    @staticmethod
    def forward(ctx, x, w, b, eps, fork=False, out=None):
        xc = x.contiguous()
        y, mean, rstd = C.layernorm_fwd(xc, w, b, eps, out=out[0] if out else None)
        ctx.save_for_backward(xc, w, mean, rstd)
        ctx.w, ctx.b, ctx.fork = w, b, fork
        ctx.set_materialize_grads(False)                 # an unused output arrives as None, not as a zero tensor
        return (y, x) if fork else y

    @staticmethod
    def backward(ctx, dy, dres=None):
        x, w, mean, rstd = ctx.saved_tensors
        if dy is None:                                   # only the residual alias was used
            return dres, None, None, None, None, None
        dy = dy.contiguous()
        wmg, wacc = _grad_target(ctx.w)
        bmg, _ = _grad_target(ctx.b)
        if wmg is not None and bmg is not None:
            dx, _, _ = C.layernorm_bwd(dy, x, w, mean, rstd, dw=wmg, db=bmg, accumulate=wacc,
                                       dres=dres)
            _grad_done(ctx.w)
            _grad_done(ctx.b)
            return dx, None, None, None, None, None
        dx, dw, db = C.layernorm_bwd(dy, x, w, mean, rstd, dres=dres)
        return dx, dw.to(w.dtype), db.to(w.dtype), None, None, None


def layernorm(x, weight, bias, eps: float = 1e-5):
    if not x.is_cuda:
        return F.layer_norm(x, (x.shape[-1],), weight, bias, eps)
    return _LayerNormFn.apply(x, weight, bias, eps, False)


def layernorm_fork(x, weight, bias, eps: float = 1e-5, out=None):
    """(LayerNorm(x), x): use the second value for the residual connection around the normalised branch.  On CUDA the
    gradient that comes back through the residual is added inside the norm's backward kernel instead of by a
    separate add.  ``out``: a contiguous CUDA tensor of x's size and dtype that receives the normalised rows (the
    input slot of a collective, for instance); nothing may keep a reference to its previous contents."""
    if not x.is_cuda:
        return layernorm(x, weight, bias, eps), x
    return _LayerNormFn.apply(x, weight, bias, eps, True, (out,) if out is not None else None)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps, fork=False, out=None):
        xc = x.contiguous()
        y, rstd = C.rmsnorm_fwd(xc, w, eps, out=out[0] if out else None)
        ctx.save_for_backward(xc, w, rstd)
        ctx.w, ctx.fork = w, fork
        ctx.set_materialize_grads(False)
        return (y, x) if fork else y

    @staticmethod
    def backward(ctx, dy, dres=None):
        x, w, rstd = ctx.saved_tensors
        if dy is None:
            return dres, None, None, None, None
        dy = dy.contiguous()
        wmg, wacc = _grad_target(ctx.w)
        if wmg is not None:
            dx, _ = C.rmsnorm_bwd(dy, x, w, rstd, dw=wmg, accumulate=wacc, dres=dres)
            _grad_done(ctx.w)
            return dx, None, None, None, None
        dx, dw = C.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
        return dx, dw.to(w.dtype), None, None, None


def rmsnorm_ref(x, weight, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()).to(x.dtype)


def rmsnorm(x, weight, eps: float = 1e-5):
    if not x.is_cuda:
        return rmsnorm_ref(x, weight, eps)
    return _RMSNormFn.apply(x, weight, eps, False)


def rmsnorm_fork(x, weight, eps: float = 1e-5, out=None):
    """(RMSNorm(x), x); see layernorm_fork."""
    if not x.is_cuda:
        return rmsnorm(x, weight, eps), x
    return _RMSNormFn.apply(x, weight, eps, True, (out,) if out is not None else None)


# ------------------------------------------------------------------------ activations
class _GeluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        return C.gelu_fwd(xc)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return C.gelu_bwd(dy.contiguous(), x)


def gelu(x):
    return _GeluFn.apply(x) if x.is_cuda else gelu_ref(x)


class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        xc = x.contiguous()
        ctx.save_for_backward(xc)
        return C.swiglu_fwd(xc)

    @staticmethod
    def backward(ctx, dy):
        (x,) = ctx.saved_tensors
        return C.swiglu_bwd(dy.contiguous(), x)


def swiglu(x):
    """``silu(x[..., :F]) * x[..., F:]`` on a fused gate/up projection of width 2F."""
    if not x.is_cuda:
        g, u = x.chunk(2, dim=-1)
        return F.silu(g) * u
    return _SwiGLUFn.apply(x)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos_offset, theta):
        ctx.args = (pos_offset, theta)
        return C.rope(x.contiguous(), pos_offset, theta, False, False)

    @staticmethod
    def backward(ctx, dy):
        pos_offset, theta = ctx.args
        return C.rope(dy.contiguous(), pos_offset, theta, True, False), None, None


def rope_ref(x, pos_offset: int, theta: float):
    B, T, H, hd = x.shape
    half = hd // 2
    inv = theta ** (-torch.arange(0, half, device=x.device, dtype=torch.float32) * 2.0 / hd)
    ang = (torch.arange(T, device=x.device, dtype=torch.float32) + pos_offset)[:, None] * inv[None, :]
    cos, sin = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


def rope(x, pos_offset: int = 0, theta: float = 500000.0):
    """Rotary embedding on [B, T, H, hd], pairing element i with i + hd/2."""
    if not x.is_cuda:
        return rope_ref(x, pos_offset, theta)
    return _RopeFn.apply(x, pos_offset, theta)


class _RopeQKVFn(torch.autograd.Function):
    """Rotates the first ``n_heads`` heads (q and k) of a fused [B, T, W] projection in place."""

    @staticmethod
    def forward(ctx, qkv, n_heads, hd, pos_offset, theta):
        ctx.args = (n_heads, hd, pos_offset, theta)
        C.rope_qkv_(qkv, n_heads, hd, pos_offset, theta, False)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, d):
        n_heads, hd, pos_offset, theta = ctx.args
        d = d.contiguous()
        C.rope_qkv_(d, n_heads, hd, pos_offset, theta, True)
        return d, None, None, None, None


def rope_qkv(qkv, n_rot_heads: int, head_dim: int, pos_offset: int = 0, theta: float = 500000.0):
    """RoPE on the q and k heads of a fused QKV projection [B, T, (Hq + 2 Hkv) * hd]."""
    if qkv.is_cuda and qkv.dtype in (torch.float32, _bf16) and qkv.is_contiguous():
        return _RopeQKVFn.apply(qkv, n_rot_heads, head_dim, pos_offset, theta)
    B, T, W = qkv.shape
    n = n_rot_heads * head_dim
    rot = rope(qkv[..., :n].reshape(B, T, n_rot_heads, head_dim), pos_offset, theta).reshape(B, T, n)
    return torch.cat([rot, qkv[..., n:]], dim=-1)


# -------------------------------------------------------------------------- embedding
class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, idx, wte, wpe, pos_offset, vocab_lo):
        idxc = idx.contiguous()
        lookup = idxc
        if vocab_lo:
            # vocabulary-parallel shard: rows outside [lo, lo + rows) read row 0 and are masked by the caller
            lookup = (idxc - vocab_lo).clamp_(0, wte.shape[0] - 1)
        out = C.embedding_fwd(lookup, wte, wpe, pos_offset)
        ctx.save_for_backward(idxc)
        ctx.wte, ctx.wpe = wte, wpe
        ctx.vocab = (vocab_lo, vocab_lo + wte.shape[0])
        return out

    @staticmethod
    def backward(ctx, dout):
        (idx,) = ctx.saved_tensors
        wte, wpe = ctx.wte, ctx.wpe
        dout = dout.contiguous()
        lo, hi = ctx.vocab
        gw = gp = None
        wmg, wacc = _grad_target(wte)
        if wmg is None:
            gw_buf = torch.zeros(wte.shape, device=wte.device, dtype=torch.float32)
        else:
            gw_buf = wmg
            if not wacc:
                gw_buf.zero_()
        gp_buf = None
        if wpe is not None:
            pmg, pacc = _grad_target(wpe)
            if pmg is None:
                gp_buf = torch.zeros(wpe.shape, device=wpe.device, dtype=torch.float32)
            else:
                gp_buf = pmg
                if not pacc:
                    gp_buf.zero_()
        C.embedding_bwd(idx, dout, gw_buf.view(wte.shape), gp_buf.view(wpe.shape) if gp_buf is not None else None,
                        lo, hi, DETERMINISTIC_EMBEDDING_GRAD)
        if wmg is None:
            gw = gw_buf.to(wte.dtype)
        else:
            _grad_done(wte)
        if wpe is not None:
            if getattr(wpe, "main_grad", None) is None:
                gp = gp_buf.to(wpe.dtype)
            else:
                _grad_done(wpe)
        return None, gw, gp, None, None


def embedding(idx, wte, wpe=None, pos_offset: int = 0, vocab_lo: int = 0):
    """Token embedding gather, optionally fused with the position-embedding add."""
    if not wte.is_cuda:
        out = F.embedding(idx - vocab_lo if vocab_lo else idx, wte)
        if wpe is not None:
            T = idx.shape[-1]
            out = out + wpe[pos_offset:pos_offset + T]
        return out
    return _EmbeddingFn.apply(idx, wte, wpe, pos_offset, vocab_lo)


# ---------------------------------------------------------------- softmax / cross entropy
class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        y = C.softmax_fwd(x.contiguous(), dim)
        ctx.save_for_backward(y)
        ctx.dim = dim
        return y

    @staticmethod
    def backward(ctx, dy):
        (y,) = ctx.saved_tensors
        return C.softmax_bwd(dy.contiguous(), y, ctx.dim), None


def softmax(x, dim: int = -1):
    return _SoftmaxFn.apply(x, dim) if x.is_cuda else torch.softmax(x, dim)


class _CrossEntropyFn(torch.autograd.Function):
    """Mean cross entropy over rows; backward scales by the upstream scalar on the device."""

    @staticmethod
    def forward(ctx, logits, targets, V):
        lc = logits.contiguous()
        rows = lc.numel() // lc.shape[-1]
        tc = targets.contiguous().view(-1)
        if tc.dtype != torch.int64:
            tc = tc.to(torch.int64)
        loss = C.xent_fused(lc, tc, V, 0.0, False, 1.0 / rows)
        ctx.save_for_backward(lc, tc)
        ctx.V, ctx.rows = V, rows
        return loss

    @staticmethod
    def backward(ctx, dloss):
        lc, tc = ctx.saved_tensors
        d = C.xent_bwd(lc, tc, dloss, ctx.V, 1.0 / ctx.rows, False)
        return d, None, None


def cross_entropy(logits, targets, vocab_size: Optional[int] = None):
    """Mean softmax cross entropy; columns >= vocab_size of ``logits`` are padding."""
    V = logits.shape[-1] if vocab_size is None else vocab_size
    if not logits.is_cuda:
        lg = logits[..., :V].reshape(-1, V).float()
        return F.cross_entropy(lg, targets.reshape(-1).long())
    return _CrossEntropyFn.apply(logits, targets, V).to(torch.float32)


class _LMHeadLossFn(torch.autograd.Function):
    """loss = mean CE(x W^T, targets) with the logits gradient written over the logits.

    The [rows, V_padded] logits tensor is produced by the tcgen05 GEMM, reduced to the
    loss and replaced by ``(softmax - onehot) / rows`` in one kernel; backward feeds it
    straight to the dgrad and wgrad GEMMs, scaled by the upstream gradient through the
    GEMM's device-side alpha.
    """

    @staticmethod
    def forward(ctx, x, w, targets, V):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        rows = x2.shape[0]
        logits = C.gemm(x2, w)[0]
        tc = targets.contiguous().view(-1)
        loss = C.xent_fused(logits, tc, V, 1.0 / rows, True, 1.0 / rows)
        ctx.save_for_backward(x2, w, logits)
        ctx.xshape = x.shape
        return loss

    @staticmethod
    def backward(ctx, dloss):
        x2, w, dlogits = ctx.saved_tensors
        alpha = dloss.reshape(1).to(torch.float32)
        dx = C.gemm(dlogits, w, False, True, alpha=alpha)[0].view(ctx.xshape)
        dw = _wgrad(dlogits, x2, w, alpha=alpha)
        return dx, dw, None, None


def lm_head_loss(x, weight, targets, vocab_size: int):
    """Fused output projection + mean cross entropy (weight: [V_padded, C])."""
    if x.is_cuda and x.dtype == _bf16:
        return _LMHeadLossFn.apply(x, weight, targets, vocab_size)
    logits = linear(x, weight)
    return cross_entropy(logits, targets, vocab_size)


# -------------------------------------------------------------------------- attention
_ATTN_IMPL = {"impl": os.environ.get("TITB200_ATTN", "native")}


def set_attention_impl(name: str) -> None:
    """'native' = the tcgen05 flash-attention kernels of this package; 'sdpa' = torch's
    scaled_dot_product_attention, kept only as the unfused baseline arm."""
    assert name in ("native", "sdpa")
    _ATTN_IMPL["impl"] = name


def attention_ref(q, k, v, scale=None):
    """softmax(mask(q k^T / sqrt(hd))) v with q [B,T,Hq,hd], k/v [B,T,Hkv,hd] (example/gpt2/net.cc:91-108)."""
    B, T, Hq, hd = q.shape
    Hkv = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    qf, kf, vf = (t.float().transpose(1, 2) for t in (q, k, v))
    if Hkv != Hq:
        kf = kf.repeat_interleave(Hq // Hkv, dim=1)
        vf = vf.repeat_interleave(Hq // Hkv, dim=1)
    att = (qf @ kf.transpose(-1, -2)) * scale
    mask = torch.ones(T, T, device=q.device, dtype=torch.bool).tril()
    att = att.masked_fill(~mask, float("-inf")).softmax(-1)
    return (att @ vf).transpose(1, 2).to(q.dtype)


class _AttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        o, lse = C.attn_fwd(q, k, v, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = C.attn_bwd(do.contiguous(), q, k, v, o, lse, ctx.scale)
        return dq, dk, dv, None


class _AttentionQKVFn(torch.autograd.Function):
    """Attention over a fused projection buffer [B, T, (Hq + 2 Hkv) * hd]: q/k/v are read in
    place and dq/dk/dv are written into one fused gradient buffer of the same layout."""

    @staticmethod
    def _views(t, Hq, Hkv, hd):
        B, T, _ = t.shape
        q = t[..., :Hq * hd].view(B, T, Hq, hd)
        k = t[..., Hq * hd:(Hq + Hkv) * hd].view(B, T, Hkv, hd)
        v = t[..., (Hq + Hkv) * hd:].view(B, T, Hkv, hd)
        return q, k, v

    @staticmethod
    def forward(ctx, qkv, Hq, Hkv, hd, scale):
        qkv = qkv.contiguous()
        q, k, v = _AttentionQKVFn._views(qkv, Hq, Hkv, hd)
        o, lse = C.attn_fwd(q, k, v, scale)
        ctx.save_for_backward(qkv, o, lse)
        ctx.args = (Hq, Hkv, hd, scale)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, o, lse = ctx.saved_tensors
        Hq, Hkv, hd, scale = ctx.args
        q, k, v = _AttentionQKVFn._views(qkv, Hq, Hkv, hd)
        dqkv = torch.empty_like(qkv)
        dq, dk, dv = _AttentionQKVFn._views(dqkv, Hq, Hkv, hd)
        C.attn_bwd(do, q, k, v, o, lse, scale, dq, dk, dv)
        return dqkv, None, None, None, None


def causal_attention_qkv(qkv, n_head: int, n_kv_head: Optional[int] = None, scale: Optional[float] = None):
    """Causal attention on a fused QKV projection [B, T, (Hq + 2 Hkv) * hd] -> [B, T, Hq, hd]."""
    Hq = n_head
    Hkv = n_kv_head if n_kv_head is not None else n_head
    hd = qkv.shape[-1] // (Hq + 2 * Hkv)
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if qkv.is_cuda and qkv.dtype == _bf16 and _ATTN_IMPL["impl"] == "native" and hd in (64, 128):
        return _AttentionQKVFn.apply(qkv, Hq, Hkv, hd, scale)
    B, T, _ = qkv.shape
    q = qkv[..., :Hq * hd].reshape(B, T, Hq, hd)
    k = qkv[..., Hq * hd:(Hq + Hkv) * hd].reshape(B, T, Hkv, hd)
    v = qkv[..., (Hq + Hkv) * hd:].reshape(B, T, Hkv, hd)
    return causal_attention(q, k, v, scale)


def causal_attention(q, k, v, scale: Optional[float] = None):
    """Causal self-attention.  q: [B, T, Hq, hd]; k, v: [B, T, Hkv, hd] (Hq % Hkv == 0).

    The tensors may be strided views of one fused projection buffer; the output is
    [B, T, Hq, hd] contiguous, i.e. already the [B, T, C] layout the next GEMM reads.
    """
    hd = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    if not q.is_cuda:
        return attention_ref(q, k, v, scale)
    if _ATTN_IMPL["impl"] == "sdpa" or q.dtype != _bf16 or hd not in (64, 128):
        Hq, Hkv = q.shape[2], k.shape[2]
        qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, scale=scale, enable_gqa=Hq != Hkv)
        return o.transpose(1, 2).contiguous()
    return _AttentionFn.apply(q, k, v, scale)


# -------------------------------------------------------------------- elementwise family
UNARY = {"neg": 0, "reciprocal": 1, "sin": 2, "cos": 3, "tanh": 4, "pow_exp": 5, "pow_base": 6, "rsqrt": 7,
         "equals_scalar": 8, "add_scalar": 9, "mul_scalar": 10, "sigmoid": 11, "copy": 12}
_SAVES_OUTPUT = {4, 11}

_UNARY_REF = {
    0: lambda x, s: -x, 1: lambda x, s: 1.0 / x, 2: lambda x, s: torch.sin(x), 3: lambda x, s: torch.cos(x),
    4: lambda x, s: torch.tanh(x), 5: lambda x, s: torch.pow(x, s), 6: lambda x, s: torch.pow(s, x),
    7: lambda x, s: torch.rsqrt(x), 8: lambda x, s: (x == s).to(x.dtype), 9: lambda x, s: x + s,
    10: lambda x, s: x * s, 11: lambda x, s: torch.sigmoid(x), 12: lambda x, s: x.clone(),
}


class _UnaryFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, s):
        xc = x.contiguous()
        y = C.unary_fwd(op, xc, s)
        ctx.save_for_backward(y if op in _SAVES_OUTPUT else xc)
        ctx.op, ctx.s = op, s
        return y

    @staticmethod
    def backward(ctx, dy):
        if ctx.op == 8:
            raise RuntimeError("EqualsScalar has no gradient")
        (saved,) = ctx.saved_tensors
        return C.unary_bwd(ctx.op, dy.contiguous(), saved, ctx.s), None, None


def unary(name: str, x, s: float = 0.0):
    op = UNARY[name]
    if not x.is_cuda or x.dtype not in (torch.float32, _bf16):
        return _UNARY_REF[op](x, s)
    return _UnaryFn.apply(x, op, float(s))


BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3}
_BINARY_REF = {0: torch.add, 1: torch.sub, 2: torch.mul, 3: torch.div}


def _reduce_to(g, shape):
    """Sum a gradient of a's shape down to b's (right-aligned) shape."""
    while g.dim() > len(shape):
        g = g.sum(0)
    for d, n in enumerate(shape):
        if n == 1 and g.shape[d] != 1:
            g = g.sum(d, keepdim=True)
    return g


class _BinaryFn(torch.autograd.Function):
    """a (op) broadcast(b) -> a's shape (infini_train/src/kernels/cpu/elementwise.cc:44-123)."""

    @staticmethod
    def forward(ctx, a, b, op):
        ac, bc = a.contiguous(), b.contiguous()
        ctx.save_for_backward(ac, bc)
        ctx.op = op
        return C.binary_fwd(op, ac, bc)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        op = ctx.op
        dy = dy.contiguous()
        if op == 0:
            da, db_full = dy, dy
        elif op == 1:
            da, db_full = dy, C.unary_fwd(0, dy, 0.0)
        elif op == 2:
            da, db_full = C.binary_fwd(2, dy, b), C.binary_fwd(2, dy, a)
        else:
            da = C.binary_fwd(3, dy, b)
            q = C.binary_fwd(3, da, b)            # dy / b^2
            db_full = C.unary_fwd(0, C.binary_fwd(2, q, a), 0.0)
        return da, _reduce_to(db_full, b.shape).reshape(b.shape), None


def binary(name: str, a, b):
    op = BINARY[name]
    if not a.is_cuda or a.dtype not in (torch.float32, _bf16) or a.dtype != b.dtype or b.dim() > a.dim():
        return _BINARY_REF[op](a, b)
    return _BinaryFn.apply(a, b, op)


class _CastFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dtype):
        ctx.src = x.dtype
        return C.cast(x.contiguous(), dtype == _bf16)

    @staticmethod
    def backward(ctx, dy):
        return C.cast(dy.contiguous(), ctx.src == _bf16), None


def cast(x, dtype):
    """dtype conversion between float32 and bfloat16 (differentiable)."""
    if x.dtype == dtype:
        return x
    if x.is_cuda and x.dtype in (torch.float32, _bf16) and dtype in (torch.float32, _bf16):
        return _CastFn.apply(x, dtype)
    return x.to(dtype)


class _TransposeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return C.transpose_last2(x.contiguous())

    @staticmethod
    def backward(ctx, dy):
        return C.transpose_last2(dy.contiguous())


def transpose(x, d0: int, d1: int):
    """Swap two axes and materialise a contiguous copy (reference Transpose semantics)."""
    nd = x.dim()
    d0, d1 = d0 % nd, d1 % nd
    if x.is_cuda and x.dtype in (torch.float32, _bf16) and {d0, d1} == {nd - 1, nd - 2}:
        return _TransposeFn.apply(x)
    return x.transpose(d0, d1).contiguous()


class _TriFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, diagonal, upper):
        ctx.args = (diagonal, upper)
        return C.tri(x.contiguous(), diagonal, upper)

    @staticmethod
    def backward(ctx, dy):
        return C.tri(dy.contiguous(), *ctx.args), None, None


def tril(x, diagonal: int = 0):
    if x.is_cuda and x.dim() == 2 and x.dtype in (torch.float32, _bf16):
        return _TriFn.apply(x, diagonal, False)
    return torch.tril(x, diagonal)


def triu(x, diagonal: int = 0):
    if x.is_cuda and x.dim() == 2 and x.dtype in (torch.float32, _bf16):
        return _TriFn.apply(x, diagonal, True)
    return torch.triu(x, diagonal)


# ----------------------------------------------------------------------------- reductions along one axis
_REDUCE_OPS = {"sum": 0, "mean": 1, "max": 2, "min": 3}


def _own_kernel_ok(x) -> bool:
    return x.is_cuda and x.dtype in (torch.float32, _bf16)


class _ReduceFn(torch.autograd.Function):
    """Mean / Sum / Max / Min over one axis (reference: infini_train/src/autograd/reduction.cc,
    kernels/cuda/reduction.cu).  Max / Min route the gradient to the selected element only."""

    @staticmethod
    def forward(ctx, x, op, dim, keepdim):
        y, idx = C.reduce_dim(x, op, dim, keepdim)
        ctx.meta = (op, dim % x.dim(), tuple(x.shape))
        ctx.idx = idx
        return y

    @staticmethod
    def backward(ctx, dy):
        op, dim, shape = ctx.meta
        scale = 1.0 / shape[dim] if op == 1 else 1.0
        return C.reduce_dim_bwd(dy, ctx.idx, list(shape), dim, scale), None, None, None


def reduce(name: str, x, dim: int, keepdim: bool = False):
    if _own_kernel_ok(x) and x.dim() >= 1:
        return _ReduceFn.apply(x, _REDUCE_OPS[name], dim, keepdim)
    if name in ("sum", "mean"):
        return getattr(torch, name)(x, dim=dim, keepdim=keepdim)
    return getattr(torch, name)(x, dim=dim, keepdim=keepdim).values


def sum_dim(x, dim: int, keepdim: bool = False):
    return reduce("sum", x, dim, keepdim)


def mean_dim(x, dim: int, keepdim: bool = False):
    return reduce("mean", x, dim, keepdim)


def max_dim(x, dim: int, keepdim: bool = False):
    return reduce("max", x, dim, keepdim)


def min_dim(x, dim: int, keepdim: bool = False):
    return reduce("min", x, dim, keepdim)


# ----------------------------------------------------------------------------- view-like ops through one gather kernel
def _contig_strides(shape):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= s
    return list(reversed(st))


class _GatherViewFn(torch.autograd.Function):
    """Materialises a strided view (sizes, strides, offset over a contiguous input).  The backward
    scatters into a zero tensor, accumulating when the view repeats elements (stride 0)."""

    @staticmethod
    def forward(ctx, x, sizes, strides, offset):
        xc = x.contiguous()
        ctx.meta = (tuple(x.shape), list(strides), offset)
        return C.gather_view(xc, list(sizes), list(strides), offset)

    @staticmethod
    def backward(ctx, dy):
        shape, strides, offset = ctx.meta
        dx = torch.zeros(shape, device=dy.device, dtype=dy.dtype)
        C.scatter_view_(dx, dy, strides, offset, accumulate=any(s == 0 for s in strides))
        return dx, None, None, None


def slice_nd(x, starts, ends, steps):
    """Per-dimension [start, end) with step (reference: infini_train/src/kernels/cuda/slice.cu)."""
    if not (_own_kernel_ok(x) and x.dim() <= 6):
        idx = tuple(slice(s, e, st) for s, e, st in zip(starts, ends, steps))
        return x[idx].contiguous()
    base = _contig_strides(x.shape)
    sizes = [(e - s + st - 1) // st for s, e, st in zip(starts, ends, steps)]
    strides = [b * st for b, st in zip(base, steps)]
    offset = sum(s * b for s, b in zip(starts, base))
    return _GatherViewFn.apply(x, sizes, strides, offset)


def split(x, split_size: int, dim: int = 0):
    """Equal chunks of ``split_size`` along ``dim`` (the last may be shorter); each a contiguous tensor."""
    dim = dim % x.dim()
    n = x.shape[dim]
    outs = []
    for s in range(0, n, split_size):
        starts = [0] * x.dim()
        ends = list(x.shape)
        starts[dim], ends[dim] = s, min(s + split_size, n)
        outs.append(slice_nd(x, starts, ends, [1] * x.dim()))
    return outs


def repeat_interleave(x, repeats: int, dim: int):
    """Each element along ``dim`` repeated ``repeats`` times in place (reference transform.cu RepeatInterleave)."""
    dim = dim % x.dim()
    if not (_own_kernel_ok(x) and x.dim() <= 5):
        return torch.repeat_interleave(x, repeats, dim=dim)
    base = _contig_strides(x.shape)
    sizes = list(x.shape[:dim + 1]) + [repeats] + list(x.shape[dim + 1:])
    strides = base[:dim + 1] + [0] + base[dim + 1:]
    out = _GatherViewFn.apply(x, sizes, strides, 0)
    shape = list(x.shape)
    shape[dim] *= repeats
    return out.view(shape)


class _StackFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, dim, *xs):
        shape = list(xs[0].shape)
        n = len(xs)
        out_shape = shape[:dim] + [n] + shape[dim:]
        out = torch.empty(out_shape, device=xs[0].device, dtype=xs[0].dtype)
        ost = _contig_strides(out_shape)
        view_strides = ost[:dim] + ost[dim + 1:]
        for i, x in enumerate(xs):
            C.scatter_view_(out, x.contiguous(), view_strides, i * ost[dim], False)
        ctx.meta = (dim, n, shape, view_strides, ost[dim])
        return out

    @staticmethod
    def backward(ctx, dy):
        dim, n, shape, view_strides, step = ctx.meta
        dyc = dy.contiguous()
        return (None,) + tuple(C.gather_view(dyc, shape, view_strides, i * step) for i in range(n))


def stack(xs, dim: int = 0):
    xs = list(xs)
    nd = xs[0].dim() + 1
    dim = dim % nd
    if all(_own_kernel_ok(x) for x in xs) and nd <= 6:
        return _StackFn.apply(dim, *xs)
    return torch.stack(xs, dim)


class _MaskFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, value):
        ctx.save_for_backward(mask)
        return C.mask_fill(x, mask, value, False)

    @staticmethod
    def backward(ctx, dy):
        (mask,) = ctx.saved_tensors
        return C.mask_fill(dy, mask, 0.0, True), None, None


def masked_fill(x, mask, value: float):
    """``mask != 0 ? value : x``; the mask tiles the trailing dimensions of ``x`` (reference transform.cu Mask)."""
    if _own_kernel_ok(x) and mask.is_cuda and x.numel() % max(1, mask.numel()) == 0 and \
            tuple(mask.shape) == tuple(x.shape[x.dim() - mask.dim():]):
        return _MaskFn.apply(x, mask, float(value))
    return x.masked_fill(mask != 0, value)


class _OuterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return C.outer_fwd(a, b)

    @staticmethod
    def backward(ctx, dy):
        a, b = ctx.saved_tensors
        da, db = C.outer_bwd(dy, a, b)
        return da, db


def outer(a, b):
    if _own_kernel_ok(a) and _own_kernel_ok(b) and a.dtype == b.dtype and a.dim() == 1 and b.dim() == 1:
        return _OuterFn.apply(a, b)
    return torch.outer(a, b)
