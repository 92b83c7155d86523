"""Parallelism: data parallel + ZeRO-1 (zero), tensor/sequence parallel (tp), pipeline (pp)."""
from .zero import DistributedOptimizer  # noqa: F401
