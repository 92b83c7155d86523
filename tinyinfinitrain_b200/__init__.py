"""tinyinfinitrain_b200 -- a Blackwell-native (sm_100a) LLM training framework.

Layers (bottom up): ``csrc/kernels`` hand-written CUDA (tcgen05 GEMM and
attention, norms, loss, optimizers, NVLink collectives) -> ``ops`` autograd
functions -> ``nn`` modules -> ``models`` (GPT-2, LLaMA-3) -> ``optim`` /
``parallel`` (DP + ZeRO-1, TP + SP, PP) -> ``data`` / ``utils`` (llm.c file
formats, tokenizer, checkpoints, timers).
"""
from . import _lib  # noqa: F401

__version__ = "0.1.0"

from . import ops  # noqa: E402,F401
from . import nn  # noqa: E402,F401
from . import optim  # noqa: E402,F401
from . import data  # noqa: E402,F401
from . import utils  # noqa: E402,F401
from . import models  # noqa: E402,F401
from . import parallel  # noqa: E402,F401
