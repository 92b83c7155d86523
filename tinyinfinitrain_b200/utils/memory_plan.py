"""Per-GPU memory plan of a training configuration, computed from the model shape and the parallel layout.

    python -m tinyinfinitrain_b200 plan --model llama3-8b --tp 4 --dp 2 --batch 2 --seq 4096
    python -m tinyinfinitrain_b200 plan --model gpt2-xl --tp 2 --pp 2 --dp 2 --batch 4 --seq 1024 --micro_batches 8

It answers "does this fit in the 180 GB of a B200, and what takes the space" before any GPU is touched.  The
byte counts follow what the framework allocates:

* parameters: bf16 copy, one per tensor- / pipeline-parallel rank's slice (replicated over data parallelism),
* main gradients: fp32, same slice (the wgrad kernels accumulate straight into this buffer),
* optimizer state: fp32 master weights + two Adam moments, divided by the data-parallel size under ZeRO-1,
* activations kept for backward, per layer and micro-batch (sequence-parallel regions hold 1/tp of the rows), times
  the number of micro-batches in flight on the stage under 1F1B (at most pp - stage),
* logits + their gradient (in place) for the vocabulary slice of the last stage, plus the fused-collective staging
  buffers of tensor parallelism.

The reference has no multi-GPU support and no planner; its TensorBuffer allocates on demand
(infini_train/src/tensor.cc:58-96).
"""
from __future__ import annotations

import argparse
import json
from dataclasses import dataclass
from typing import Dict

HBM_BYTES = 183_359 * 2**20       # what nvidia-smi reports for a B200 (MiB -> bytes)


@dataclass
class Shape:
    family: str          # "gpt2" | "llama3"
    n_layer: int
    n_head: int
    n_kv_head: int
    n_embd: int
    ffn: int
    vocab: int           # padded vocabulary rows actually allocated
    block_size: int


def shape_of(model) -> Shape:
    """``model``: a preset name (``gpt2``, ``gpt2-xl``, ``llama3-8b`` ...) or a GPT2Config / LLaMA3Config."""
    from ..models import GPT2_PRESETS
    from ..models.gpt2 import GPT2Config
    from ..models.llama3 import LLAMA3_PRESETS, LLaMA3Config

    c = model
    if isinstance(model, str):
        if model not in GPT2_PRESETS and model not in LLAMA3_PRESETS:
            raise KeyError(f"unknown model {model!r}")
        c = GPT2_PRESETS.get(model) or LLAMA3_PRESETS[model]
    if isinstance(c, GPT2Config):
        return Shape("gpt2", c.n_layer, c.n_head, c.n_head, c.n_embd, 4 * c.n_embd, c.padded_vocab_size, c.block_size)
    if isinstance(c, LLaMA3Config):
        vocab = getattr(c, "padded_vocab_size", None) or c.vocab_size
        return Shape("llama3", c.n_layer, c.n_head, c.n_kv_head, c.n_embd, c.ffn_dim, vocab, c.block_size)
    raise TypeError(f"cannot plan for {type(model).__name__}")


def layer_params(s: Shape) -> int:
    C = s.n_embd
    hd = C // s.n_head
    qkv = C * (s.n_head + 2 * s.n_kv_head) * hd
    if s.family == "gpt2":   # weights + biases of c_attn, c_proj, c_fc, mlp.c_proj; two LayerNorms
        return (qkv + (s.n_head + 2 * s.n_kv_head) * hd) + (C * C + C) + (C * s.ffn + s.ffn) + (s.ffn * C + C) + 4 * C
    return qkv + C * C + C * 2 * s.ffn + s.ffn * C + 2 * C       # no biases, gate and up fused, two RMSNorms


def total_params(s: Shape) -> int:
    C = s.n_embd
    emb = s.vocab * C + (s.block_size * C if s.family == "gpt2" else 0)
    head = 0 if s.family == "gpt2" else s.vocab * C            # GPT-2 ties lm_head to wte
    final_norm = 2 * C if s.family == "gpt2" else C
    return emb + head + final_norm + s.n_layer * layer_params(s)


def plan(model, tp: int = 1, pp: int = 1, dp: int = 1, batch: int = 8, seq: int = 1024, micro_batches: int = 1,
         zero_stage: int = 1, stage: int = 0) -> Dict:
    """Bytes per GPU for pipeline stage ``stage`` (0 = first).  ``batch`` is the micro-batch size per data-parallel rank."""
    s = shape_of(model)
    C, hd = s.n_embd, s.n_embd // s.n_head
    layers = s.n_layer // pp + (1 if stage < s.n_layer % pp else 0)
    first, last = stage == 0, stage == pp - 1
    # parameters of this rank: the matrices are split over tp, norms (and GPT-2's row-parallel biases) are replicated
    per_layer = layer_params(s)
    norms = (4 * C + 2 * C if s.family == "gpt2" else 2 * C)   # GPT-2: two LayerNorms + the two row-parallel biases
    layer_local = (per_layer - norms) / tp + norms
    n_local = layers * layer_local
    if first:
        n_local += s.vocab * C / tp + (s.block_size * C if s.family == "gpt2" else 0)
    if last:
        n_local += (2 * C if s.family == "gpt2" else C)
        if s.family != "gpt2" or not first:                      # untied head, or the tied copy a last stage keeps
            n_local += s.vocab * C / tp
    params = 2 * n_local
    grads = 4 * n_local
    opt = 12 * n_local / (dp if zero_stage >= 1 else 1)
    # activations saved per layer and micro-batch (bf16 unless noted): rows = batch * seq tokens
    rows = batch * seq
    sp_rows = rows / tp                                          # residual stream and norm outputs are sequence-sharded
    qkv_w = (s.n_head + 2 * s.n_kv_head) * hd / tp
    if s.family == "gpt2":
        mlp = 2 * rows * s.ffn / tp * 2                          # pre-activation and GELU output
    else:
        mlp = (rows * 2 * s.ffn / tp + rows * s.ffn / tp) * 2    # gate|up and the SwiGLU product
    per_layer_act = (
        2 * sp_rows * C * 2                                      # the two norm inputs (residual stream)
        + (2 * rows * C * 2 if tp > 1 else 2 * sp_rows * C * 2)  # gathered norm outputs kept for the wgrad GEMMs
        + rows * qkv_w * 2                                       # fused q | k | v
        + rows * (s.n_head / tp) * hd * 2                        # attention output
        + rows * (s.n_head / tp) * 4                             # log-sum-exp per (token, head), fp32
        + mlp
        + 4 * sp_rows * 4                                        # mean / rstd of the two norms, fp32
    )
    in_flight = max(1, min(micro_batches, pp - stage))
    acts = layers * per_layer_act * in_flight
    logits = (rows * (s.vocab / tp) * 2 + sp_rows * C * 2) if last else 0
    staging = 0
    if tp > 1:                                                   # gathered-activation and reduce-scatter receive buffers
        staging = rows * C * 2 + rows * max(C, s.ffn / tp) * 2
    attn_tmp = rows * (s.n_head / tp) * hd * 4                   # fp32 dQ accumulator of the attention backward
    total = params + grads + opt + acts + logits + staging + attn_tmp
    return {
        "model": model if isinstance(model, str) else type(model).__name__,
        "layout": {"tp": tp, "pp": pp, "dp": dp, "stage": stage, "zero_stage": zero_stage},
        "micro_batch": batch, "seq": seq, "micro_batches": micro_batches, "layers_on_stage": layers,
        "parameters_total": total_params(s), "parameters_on_rank": int(n_local),
        "bytes": {"parameters_bf16": int(params), "main_gradients_fp32": int(grads), "optimizer_state_fp32": int(opt),
                  "activations": int(acts), "logits": int(logits), "tp_staging": int(staging),
                  "attention_backward_scratch": int(attn_tmp), "total": int(total)},
        "gib_total": round(total / 2**30, 2), "fits_b200": bool(total < 0.92 * HBM_BYTES),
        "fraction_of_hbm": round(total / HBM_BYTES, 3),
    }


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="tinyinfinitrain_b200 plan", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="gpt2")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--dp", type=int, default=1)
    ap.add_argument("--batch", type=int, default=8, help="micro-batch per data-parallel rank")
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--micro_batches", type=int, default=1)
    ap.add_argument("--zero_stage", type=int, default=1)
    a = ap.parse_args(argv)
    out = [plan(a.model, a.tp, a.pp, a.dp, a.batch, a.seq, a.micro_batches, a.zero_stage, st) for st in range(a.pp)]
    print(json.dumps(out if a.pp > 1 else out[0], indent=1))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
