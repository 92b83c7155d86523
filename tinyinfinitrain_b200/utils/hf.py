"""Weights from Hugging Face ``transformers`` models into this package's GPT-2 / LLaMA-3 models.

The reference's ``GPT2::FromPretrained`` aborts (example/gpt2/net.cc:223-226); here ``FromPretrained`` accepts a
local directory (or a cached model name) that ``transformers`` can open without network access.  Layout notes:
GPT-2 checkpoints store linear weights as ``Conv1D`` ([in, out]) and are transposed on the way in; LLaMA's separate
q / k / v and gate / up projections are concatenated by rows into the fused ``c_attn`` and ``c_fc`` weights.
"""
from __future__ import annotations

import torch


def gpt2_from_hf(hf_model, device=None, dtype=torch.float32):
    from ..models.gpt2 import GPT2, GPT2Config

    hc = hf_model.config
    cfg = GPT2Config(block_size=hc.n_positions, vocab_size=hc.vocab_size, n_layer=hc.n_layer, n_head=hc.n_head,
                     n_embd=hc.n_embd)
    model = GPT2(cfg, device=device, dtype=dtype, seed=None)
    src = hf_model.state_dict()
    own = model.StateDict()
    with torch.no_grad():
        own["transformer.wte.weight"][:cfg.vocab_size].copy_(src["transformer.wte.weight"])
        own["transformer.wte.weight"][cfg.vocab_size:].zero_()
        own["transformer.wpe.weight"].copy_(src["transformer.wpe.weight"])
        for l in range(cfg.n_layer):
            p = f"transformer.h.{l}."
            for name in ("ln_1.weight", "ln_1.bias", "ln_2.weight", "ln_2.bias", "attn.c_attn.bias", "attn.c_proj.bias",
                         "mlp.c_fc.bias", "mlp.c_proj.bias"):
                own[p + name].copy_(src[p + name])
            for name in ("attn.c_attn.weight", "attn.c_proj.weight", "mlp.c_fc.weight", "mlp.c_proj.weight"):
                own[p + name].copy_(src[p + name].t())          # Conv1D [in, out] -> Linear [out, in]
        own["transformer.ln_f.weight"].copy_(src["transformer.ln_f.weight"])
        own["transformer.ln_f.bias"].copy_(src["transformer.ln_f.bias"])
    return model


def llama3_from_hf(hf_model, device=None, dtype=torch.float32):
    from ..models.llama3 import LLaMA3, LLaMA3Config

    hc = hf_model.config
    theta = getattr(hc, "rope_theta", None)
    if theta is None:
        theta = (getattr(hc, "rope_parameters", None) or {}).get("rope_theta", 500000.0)
    cfg = LLaMA3Config(block_size=hc.max_position_embeddings, vocab_size=hc.vocab_size, n_layer=hc.num_hidden_layers,
                       n_head=hc.num_attention_heads, n_kv_head=hc.num_key_value_heads, n_embd=hc.hidden_size,
                       ffn_dim=hc.intermediate_size, norm_eps=hc.rms_norm_eps, rope_theta=float(theta))
    model = LLaMA3(cfg, device=device, dtype=dtype, seed=None)
    src = hf_model.state_dict()
    own = model.StateDict()
    with torch.no_grad():
        wte = own["transformer.wte.weight"]
        wte[:cfg.vocab_size].copy_(src["model.embed_tokens.weight"])
        wte[cfg.vocab_size:].zero_()
        head = src.get("lm_head.weight", src["model.embed_tokens.weight"])    # tied checkpoints carry no lm_head
        own["lm_head.weight"][:cfg.vocab_size].copy_(head)
        own["lm_head.weight"][cfg.vocab_size:].zero_()
        own["transformer.ln_f.weight"].copy_(src["model.norm.weight"])
        for l in range(cfg.n_layer):
            p, q = f"transformer.h.{l}.", f"model.layers.{l}."
            own[p + "attn.c_attn.weight"].copy_(torch.cat([src[q + "self_attn.q_proj.weight"],
                                                           src[q + "self_attn.k_proj.weight"],
                                                           src[q + "self_attn.v_proj.weight"]]))
            own[p + "attn.c_proj.weight"].copy_(src[q + "self_attn.o_proj.weight"])
            own[p + "mlp.c_fc.weight"].copy_(torch.cat([src[q + "mlp.gate_proj.weight"], src[q + "mlp.up_proj.weight"]]))
            own[p + "mlp.c_proj.weight"].copy_(src[q + "mlp.down_proj.weight"])
            own[p + "ln_1.weight"].copy_(src[q + "input_layernorm.weight"])
            own[p + "ln_2.weight"].copy_(src[q + "post_attention_layernorm.weight"])
    return model


def from_pretrained(path_or_name: str, device=None, dtype=torch.float32):
    """Opens a GPT-2 or LLaMA checkpoint with ``transformers`` (local files only) and converts it."""
    try:
        from transformers import AutoModelForCausalLM
    except ImportError as e:  # pragma: no cover
        raise NotImplementedError("FromPretrained needs the transformers package; use FromLLMC with an llm.c file") from e
    hf = AutoModelForCausalLM.from_pretrained(path_or_name, local_files_only=True)
    kind = hf.config.model_type
    if kind == "gpt2":
        return gpt2_from_hf(hf, device, dtype)
    if kind == "llama":
        return llama3_from_hf(hf, device, dtype)
    raise ValueError(f"unsupported model type {kind!r}")
