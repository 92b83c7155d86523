"""Baseline configuration 1: GPT-2 small on CPU, fp32, batch 4 x seq 64, 10 Adam steps (lr 1e-4), uniform token ids
with seed 42, N(0, 0.02) weights.  The reference cannot be built, so the oracle is an independent implementation of
the same model from stock PyTorch modules (baseline/library_gpt2.py) started from the same weights: logits, loss and
the ten-step loss trajectory must agree.  The run uses all 12 layers; TITB200_CONFIG1_LAYERS=2 shortens it for a quick
local check."""
import os
import sys

import torch

import tinyinfinitrain_b200 as tit
from tinyinfinitrain_b200.models import GPT2, GPT2Config

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from baseline.library_gpt2 import LibraryGPT2  # noqa: E402


def _copy_weights(src: GPT2, dst: LibraryGPT2) -> None:
    """Library names (h.0.c_attn, h.0.mlp_proj ...) -> this package's StateDict names (transformer.h.0.attn.c_attn ...)."""
    sd = src.StateDict()
    sub = {"c_attn": "attn.c_attn", "c_proj": "attn.c_proj", "c_fc": "mlp.c_fc", "mlp_proj": "mlp.c_proj"}
    with torch.no_grad():
        for name, p in dst.named_parameters():
            parts = name.split(".")
            if parts[0] == "h":
                parts[2] = sub.get(parts[2], parts[2])
            p.copy_(sd["transformer." + ".".join(parts)])


def test_ten_adam_steps_match_an_independent_implementation():
    L = int(os.environ.get("TITB200_CONFIG1_LAYERS", "12"))
    cfg = GPT2Config(n_layer=L)          # 12 heads, d_model 768, block 1024, vocab 50257 padded to 50304
    assert (cfg.n_head, cfg.n_embd, cfg.block_size, cfg.vocab_size, cfg.padded_vocab_size) == (12, 768, 1024, 50257, 50304)
    ours = GPT2(cfg, device="cpu", dtype=torch.float32, seed=42)
    lib = LibraryGPT2(cfg.vocab_size, cfg.padded_vocab_size, cfg.block_size, L, cfg.n_head, cfg.n_embd)
    _copy_weights(ours, lib)
    g = torch.Generator().manual_seed(42)
    idx = torch.randint(0, cfg.vocab_size, (4, 64), generator=g)
    tgt = torch.randint(0, cfg.vocab_size, (4, 64), generator=g)

    with torch.no_grad():
        logits = ours(idx)
        x = lib.wte(idx) + lib.wpe(torch.arange(64))
        for b in lib.h:
            x = b(x)
        ref_logits = torch.nn.functional.linear(lib.ln_f(x), lib.wte.weight)[..., :cfg.vocab_size]
    assert logits.shape == (4, 64, 50257)
    assert torch.allclose(logits, ref_logits, atol=2e-4, rtol=1e-4)

    opt = tit.optim.Adam(ours.parameters(), learning_rate=1e-4)
    ropt = torch.optim.Adam(lib.parameters(), lr=1e-4, betas=(0.9, 0.999), eps=1e-8)
    ours_l, ref_l = [], []
    for _ in range(10):
        opt.ZeroGrad()
        _, loss = ours(idx, tgt)
        loss.backward()
        opt.Step()
        ropt.zero_grad()
        rl = lib(idx, tgt)
        rl.backward()
        ropt.step()
        ours_l.append(float(loss.detach()))
        ref_l.append(float(rl))
    assert abs(ours_l[0] - 10.98) < 0.2                       # ~ ln(50257) + init spread
    assert ours_l[-1] < ours_l[0] - 1.0                       # the same batch ten times: the loss falls
    assert max(abs(a - b) for a, b in zip(ours_l, ref_l)) < 5e-3, (ours_l, ref_l)
