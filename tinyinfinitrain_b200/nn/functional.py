"""The reference's ``nn::function`` namespace (infini_train/include/nn/functional.h:23-168)."""
from __future__ import annotations

import torch

from .. import ops


def Tril(x, diagonal: int = 0):
    return ops.tril(x, diagonal)


def Triu(x, diagonal: int = 0):
    return ops.triu(x, diagonal)


def Ones(dims, dtype=torch.float32, device=None):
    return torch.ones(*dims, dtype=dtype, device=device)


def Reciprocal(x):
    return ops.unary("reciprocal", x)


def Sin(x):
    return ops.unary("sin", x)


def Cos(x):
    return ops.unary("cos", x)


def Tanh(x):
    return ops.unary("tanh", x)


def Pow(a, b):
    """Pow(tensor, exponent) or Pow(base, tensor)."""
    if isinstance(a, torch.Tensor):
        return ops.unary("pow_exp", a, float(b))
    return ops.unary("pow_base", b, float(a))


def Rsqrt(x):
    return ops.unary("rsqrt", x)


def Mean(x, dim: int, keep_dim: bool = False):
    return ops.mean_dim(x, dim, keep_dim)


def Sum(x, dim: int, keep_dim: bool = False):
    return ops.sum_dim(x, dim, keep_dim)


def Max(x, dim: int, keep_dim: bool = False):
    return ops.max_dim(x, dim, keep_dim)


def Min(x, dim: int, keep_dim: bool = False):
    return ops.min_dim(x, dim, keep_dim)


def Sigmoid(x):
    return ops.unary("sigmoid", x)


def Softmax(x, dim: int = -1):
    return ops.softmax(x, dim)


def Slice(x, starts, ends, steps):
    return ops.slice_nd(x, list(starts), list(ends), list(steps))


def Stack(tensors, dim: int = 0):
    return ops.stack(list(tensors), dim)
