"""Operator layer: autograd functions over the sm_100a kernels (see functional.py)."""
from .functional import (  # noqa: F401
    EPI_BIAS, EPI_BIAS_GELU, EPI_BIAS_RESIDUAL, EPI_DGELU, EPI_NONE,
    attention_ref, binary, cast, causal_attention, causal_attention_qkv, cross_entropy, embedding, gelu, gelu_ref, layernorm, layernorm_fork, linear,
    lm_head_loss, matmul, mlp_gelu, rmsnorm, rmsnorm_fork, rmsnorm_ref, rope, rope_qkv, rope_ref, set_attention_impl, softmax, swiglu,
    transpose, tril, triu, unary,
    masked_fill, max_dim, mean_dim, min_dim, outer, reduce, repeat_interleave, slice_nd, split, stack, sum_dim,
)
