"""Optimizers: reference-API SGD/Adam and the flat mixed-precision Adam."""
from .optimizers import SGD, Adam, FlatParams, MixedPrecisionAdam, Optimizer  # noqa: F401
from .schedule import LRScheduler, constant, warmup_cosine  # noqa: F401

optimizers = __import__(__name__ + ".optimizers", fromlist=["*"])  # `optim.optimizers.Adam`, as in the reference
