"""Parameter initialisers with the reference's host-RNG semantics.

Reference: infini_train/include/nn/init.h:12-49, src/nn/init.cc:24-245.  Values
are drawn on the host by the C++ core (std::mt19937 + libstdc++ distributions)
and copied to the tensor's device and dtype.  ``generator`` is an integer
seed: like the reference's by-value ``std::optional<std::mt19937>``, a seeded
call always starts from the beginning of that seed's stream; without it the
process-wide generator (``manual_seed``) advances.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from .._lib import C


def manual_seed(seed: int) -> None:
    C.rng_seed(int(seed))


def _host_like(t: torch.Tensor) -> torch.Tensor:
    return torch.empty(t.shape, dtype=torch.float32)


def _assign(t: torch.Tensor, host: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        t.copy_(host.to(device=t.device, dtype=t.dtype))
    return t


def Normal(t: torch.Tensor, mean: float = 0.0, std: float = 1.0, generator: Optional[int] = None) -> torch.Tensor:
    h = _host_like(t)
    C.rng_normal_(h, mean, std, generator)
    return _assign(t, h)


def Uniform(t: torch.Tensor, a: float = 0.0, b: float = 1.0, generator: Optional[int] = None) -> torch.Tensor:
    h = _host_like(t)
    C.rng_uniform_(h, a, b, generator)
    return _assign(t, h)


def Ones(t: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        return t.fill_(1.0)


def Zeros(t: torch.Tensor) -> torch.Tensor:
    with torch.no_grad():
        return t.zero_()


def CalculateFanInAndFanOut(t: torch.Tensor) -> Tuple[int, int]:
    if t.dim() < 2:
        raise ValueError("Fan in and fan out can not be computed for tensor with fewer than 2 dimensions")
    rf = 1
    for d in t.shape[2:]:
        rf *= d
    return t.shape[1] * rf, t.shape[0] * rf


def CalculateGain(nonlinearity: str = "leaky_relu", param: Optional[float] = None) -> float:
    if nonlinearity in ("linear", "sigmoid", "conv1d", "conv2d", "conv3d"):
        return 1.0
    if nonlinearity == "tanh":
        return 5.0 / 3.0
    if nonlinearity == "relu":
        return math.sqrt(2.0)
    if nonlinearity == "leaky_relu":
        a = 0.01 if param is None else param
        return math.sqrt(2.0 / (1.0 + a * a))
    raise ValueError(f"unsupported nonlinearity {nonlinearity}")


def KaimingUniform(t: torch.Tensor, a: float = 0.0, mode: str = "fan_in", nonlinearity: str = "leaky_relu",
                   generator: Optional[int] = None) -> torch.Tensor:
    fan_in, fan_out = CalculateFanInAndFanOut(t)
    fan = fan_in if mode == "fan_in" else fan_out
    bound = math.sqrt(3.0) * CalculateGain(nonlinearity, a) / math.sqrt(fan)
    return Uniform(t, -bound, bound, generator)


def Arange(start: int, end: int, dtype=torch.int64, device=None) -> torch.Tensor:
    return torch.arange(start, end, dtype=dtype, device=device)
