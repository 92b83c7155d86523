"""Layers: Linear, Embedding, LayerNorm, RMSNorm, CrossEntropyLoss, Sigmoid, containers.

Reference: infini_train/include/nn/modules/{linear,sparse,normalization,loss,
activations,container}.h.  Parameter names (``weight``, ``bias``) and the
default initialisation follow the reference: Linear = KaimingUniform(a=sqrt(5))
and U(+-1/sqrt(fan_in)) (src/nn/modules/linear.cc:33-40), Embedding = N(0,1)
(sparse.cc:22-26), LayerNorm = ones/zeros (normalization.cc:25-30).
"""
from __future__ import annotations

import math
from typing import Iterable, Optional

import torch

from .. import ops
from . import init
from .module import Module


class Linear(Module):
    kType = "Linear"
    kParamWeightName = "weight"
    kParamBiasName = "bias"

    def __init__(self, in_features: int, out_features: int, bias: bool = True, device=None, dtype=torch.float32):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        self.bias = torch.nn.Parameter(torch.empty(out_features, device=device, dtype=dtype)) if bias else None
        self.ResetParameters()

    def ResetParameters(self) -> None:
        init.KaimingUniform(self.weight, a=math.sqrt(5.0))
        if self.bias is not None:
            fan_in, _ = init.CalculateFanInAndFanOut(self.weight)
            bound = 1.0 / math.sqrt(fan_in) if fan_in > 0 else 0.0
            init.Uniform(self.bias, -bound, bound)

    def forward(self, x, residual=None):
        return ops.linear(x, self.weight, self.bias, residual)


class Embedding(Module):
    kType = "Embedding"
    kParamWeightName = "weight"

    def __init__(self, num_embeddings: int, embedding_dim: int, device=None, dtype=torch.float32):
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = torch.nn.Parameter(torch.empty(num_embeddings, embedding_dim, device=device, dtype=dtype))
        self.ResetParameters()

    def ResetParameters(self) -> None:
        init.Normal(self.weight, 0.0, 1.0)

    def forward(self, idx):
        return ops.embedding(idx, self.weight)


class LayerNorm(Module):
    kType = "LayerNorm"
    kParamWeightName = "weight"
    kParamBiasName = "bias"

    def __init__(self, normalized_shape, eps: float = 1e-5, device=None, dtype=torch.float32):
        super().__init__()
        if isinstance(normalized_shape, Iterable):
            normalized_shape = list(normalized_shape)[-1]
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(normalized_shape, device=device, dtype=dtype))
        self.bias = torch.nn.Parameter(torch.zeros(normalized_shape, device=device, dtype=dtype))

    def ResetParameters(self) -> None:
        init.Ones(self.weight)
        init.Zeros(self.bias)

    def forward(self, x):
        return ops.layernorm(x, self.weight, self.bias, self.eps)

    def fork(self, x, out=None):
        """(self(x), x) for a pre-norm residual block: pass the second value to the residual connection.  ``out``
        (optional) receives the normalised rows, see ``ops.layernorm_fork``."""
        return ops.layernorm_fork(x, self.weight, self.bias, self.eps, out=out)


class RMSNorm(Module):
    kType = "RMSNorm"
    kParamWeightName = "weight"

    def __init__(self, dim: int, eps: float = 1e-5, device=None, dtype=torch.float32):
        super().__init__()
        self.eps = eps
        self.weight = torch.nn.Parameter(torch.ones(dim, device=device, dtype=dtype))

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)

    def fork(self, x, out=None):
        """(self(x), x) for a pre-norm residual block: pass the second value to the residual connection.  ``out``
        (optional) receives the normalised rows, see ``ops.layernorm_fork``."""
        return ops.rmsnorm_fork(x, self.weight, self.eps, out=out)


class CrossEntropyLoss(Module):
    kType = "CrossEntropyLoss"

    def __init__(self, vocab_size: Optional[int] = None):
        super().__init__()
        self.vocab_size = vocab_size

    def forward(self, logits, target):
        return ops.cross_entropy(logits, target, self.vocab_size)


class Sigmoid(Module):
    kType = "Sigmoid"

    def forward(self, x):
        return ops.unary("sigmoid", x)


class Sequential(Module):
    """Children are keyed "0", "1", ... and run in order (container.h:11-17)."""

    kType = "Sequential"

    def __init__(self, *layers: Module):
        super().__init__()
        for i, layer in enumerate(layers):
            self.add_module(str(i), layer)

    def __len__(self):
        return len(self._modules)

    def __iter__(self):
        return iter(self._modules.values())

    def __getitem__(self, i: int):
        return self._modules[str(i)]

    def forward(self, *xs):
        out = xs
        for layer in self._modules.values():
            out = layer(*out)
            if not isinstance(out, (tuple, list)):
                out = (out,)
        return out[0] if len(out) == 1 else out


class ModuleDict(Module):
    """Named children with no forward of their own (container.h:19-23)."""

    kType = "ModuleDict"

    def __init__(self, modules: Optional[dict] = None):
        super().__init__()
        for k, v in (modules or {}).items():
            self.add_module(k, v)

    def __getitem__(self, k: str):
        return self._modules[k]

    def __contains__(self, k: str):
        return k in self._modules

    def keys(self):
        return self._modules.keys()

    def forward(self, *a, **k):
        raise RuntimeError("Not implemented: ModuleDict has no Forward")
