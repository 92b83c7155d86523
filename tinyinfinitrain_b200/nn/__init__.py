"""Neural-network layer API with the reference's names (``nn::Module``, ``nn::Linear``, ...)."""
from . import functional, init  # noqa: F401
from . import functional as function  # noqa: F401  (reference namespace name)
from .module import Module  # noqa: F401
from .modules import (  # noqa: F401
    CrossEntropyLoss, Embedding, LayerNorm, Linear, ModuleDict, RMSNorm, Sequential, Sigmoid,
)
