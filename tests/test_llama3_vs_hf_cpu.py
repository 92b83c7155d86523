"""LLaMA-3 model math against an independent implementation (Hugging Face ``LlamaForCausalLM``, when the
``transformers`` package is importable) on CPU in fp32: RMSNorm, rotary embedding (theta 500000, element i paired with
i + hd/2), grouped-query attention, SwiGLU and the untied head.  Same weights in, logits and loss must agree."""
import pytest
import torch

from tinyinfinitrain_b200.models import LLaMA3, LLaMA3Config

transformers = pytest.importorskip("transformers")


def _hf_from(ours: LLaMA3, cfg: LLaMA3Config):
    from transformers import LlamaConfig, LlamaForCausalLM

    kw = dict(vocab_size=cfg.vocab_size, hidden_size=cfg.n_embd, intermediate_size=cfg.ffn_dim,
              num_hidden_layers=cfg.n_layer, num_attention_heads=cfg.n_head, num_key_value_heads=cfg.n_kv_head,
              max_position_embeddings=cfg.block_size, rms_norm_eps=cfg.norm_eps, tie_word_embeddings=False,
              attention_bias=False, mlp_bias=False, attn_implementation="eager")
    try:
        hc = LlamaConfig(rope_theta=cfg.rope_theta, **kw)
    except TypeError:
        hc = LlamaConfig(rope_parameters={"rope_type": "default", "rope_theta": cfg.rope_theta}, **kw)
    hf = LlamaForCausalLM(hc).float().eval()
    sd = ours.StateDict()
    hd, Hq, Hkv, F = cfg.head_dim, cfg.n_head, cfg.n_kv_head, cfg.ffn_dim
    new = {"model.embed_tokens.weight": sd["transformer.wte.weight"][:cfg.vocab_size],
           "model.norm.weight": sd["transformer.ln_f.weight"], "lm_head.weight": sd["lm_head.weight"][:cfg.vocab_size]}
    for l in range(cfg.n_layer):
        p, q = f"transformer.h.{l}.", f"model.layers.{l}."
        qkv = sd[p + "attn.c_attn.weight"]                   # rows: [q | k | v]
        new[q + "self_attn.q_proj.weight"] = qkv[:Hq * hd]
        new[q + "self_attn.k_proj.weight"] = qkv[Hq * hd:(Hq + Hkv) * hd]
        new[q + "self_attn.v_proj.weight"] = qkv[(Hq + Hkv) * hd:]
        new[q + "self_attn.o_proj.weight"] = sd[p + "attn.c_proj.weight"]
        fc = sd[p + "mlp.c_fc.weight"]                       # rows: [gate | up]
        new[q + "mlp.gate_proj.weight"], new[q + "mlp.up_proj.weight"] = fc[:F], fc[F:]
        new[q + "mlp.down_proj.weight"] = sd[p + "mlp.c_proj.weight"]
        new[q + "input_layernorm.weight"] = sd[p + "ln_1.weight"]
        new[q + "post_attention_layernorm.weight"] = sd[p + "ln_2.weight"]
    missing, unexpected = hf.load_state_dict({k: v.detach().clone() for k, v in new.items()}, strict=False)
    assert not unexpected and all("rotary" in m or "inv_freq" in m for m in missing), (missing, unexpected)
    return hf


def test_llama3_logits_and_loss_match_huggingface():
    cfg = LLaMA3Config(block_size=64, vocab_size=320, n_layer=2, n_head=8, n_kv_head=2, n_embd=64, ffn_dim=176)
    ours = LLaMA3(cfg, device="cpu", dtype=torch.float32, seed=42)
    with torch.no_grad():      # non-trivial norm gains so that RMSNorm's weight is exercised
        for n, p in ours.named_parameters():
            if n.endswith("ln_1.weight") or n.endswith("ln_2.weight") or n.endswith("ln_f.weight"):
                p.add_(0.1 * torch.randn_like(p))
    hf = _hf_from(ours, cfg)
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, cfg.vocab_size, (3, 48), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (3, 48), generator=g)
    with torch.no_grad():
        logits, loss = ours(idx, tgt)
        ref = hf(input_ids=idx).logits
    assert torch.allclose(logits, ref, atol=2e-4, rtol=1e-4), (logits - ref).abs().max()
    ref_loss = torch.nn.functional.cross_entropy(ref.reshape(-1, cfg.vocab_size), tgt.reshape(-1))
    assert abs(float(loss) - float(ref_loss)) < 1e-4
