"""Parallelism: data parallel + ZeRO-1 (zero), tensor/sequence parallel (tp, fused_tp), pipeline (pp), standalone
symmetric-memory collectives (collectives)."""
from . import mesh, pp, tp  # noqa: F401
from .collectives import SymmCollective  # noqa: F401
from .param_gather import GatheredWeightLinear, RowShardedAdam  # noqa: F401
from .mesh import ParallelMesh, init_mesh  # noqa: F401
from .pp import PipelineStage, one_f_one_b_order, partition_layers  # noqa: F401
from .tp import (  # noqa: F401
    ColumnParallelLinear, RowParallelLinear, TPComm, VocabParallelEmbedding, sync_sequence_parallel_grads,
    vocab_parallel_lm_head_loss,
)
from .zero import AllReduceOptimizer, DistributedOptimizer  # noqa: F401
