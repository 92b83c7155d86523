"""LLaMA-3 family (RMSNorm, RoPE, grouped-query attention, SwiGLU, untied lm_head).

The reference tree has no LLaMA-3 model -- only the LLaMA-3 dataset and tokenizer magic
numbers (example/common/tiny_shakespeare_dataset.cc:29, tokenizer.cc:15-31); the
architecture follows the published LLaMA-3 description and llm.c's ``train_llama3.py``
parameter naming so that the checkpoint layout of ``csrc/core/llmc_io.h`` maps 1:1:
``transformer.h.N.{ln_1, attn.c_attn, attn.c_proj, ln_2, mlp.c_fc, mlp.c_proj}.weight``.

Per block the GPU path runs: RMSNorm, fused QKV GEMM, in-place RoPE on the q|k heads of the
QKV buffer, GQA flash attention reading q/k/v in place (kv heads are never expanded),
output GEMM (+residual), RMSNorm, gate|up GEMM, SwiGLU, down GEMM (+residual).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import nn, ops
from ..nn import init


@dataclass
class LLaMA3Config:
    block_size: int = 8192
    vocab_size: int = 128256
    n_layer: int = 16
    n_head: int = 32
    n_kv_head: int = 8
    n_embd: int = 2048
    ffn_dim: int = 8192
    norm_eps: float = 1e-5
    rope_theta: float = 500000.0

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head


LLAMA3_PRESETS = {
    "llama3-1b": LLaMA3Config(n_layer=16, n_head=32, n_kv_head=8, n_embd=2048, ffn_dim=8192),
    "llama3-8b": LLaMA3Config(n_layer=32, n_head=32, n_kv_head=8, n_embd=4096, ffn_dim=14336),
}


class LLaMA3Attention(nn.Module):
    kType = "CausalSelfAttention"

    def __init__(self, cfg: LLaMA3Config, device=None, dtype=torch.float32):
        super().__init__()
        self.cfg = cfg
        hd = cfg.head_dim
        self.c_attn = nn.Linear(cfg.n_embd, (cfg.n_head + 2 * cfg.n_kv_head) * hd, bias=False, device=device, dtype=dtype)
        self.c_proj = nn.Linear(cfg.n_embd, cfg.n_embd, bias=False, device=device, dtype=dtype)

    def forward(self, x, residual=None, pos_offset: int = 0):
        cfg = self.cfg
        B, T, Cdim = x.shape
        qkv = self.c_attn(x)
        qkv = ops.rope_qkv(qkv, cfg.n_head + cfg.n_kv_head, cfg.head_dim, pos_offset, cfg.rope_theta)
        y = ops.causal_attention_qkv(qkv, cfg.n_head, cfg.n_kv_head).reshape(B, T, Cdim)
        return self.c_proj(y, residual)


class LLaMA3MLP(nn.Module):
    kType = "MLP"

    def __init__(self, cfg: LLaMA3Config, device=None, dtype=torch.float32):
        super().__init__()
        self.c_fc = nn.Linear(cfg.n_embd, 2 * cfg.ffn_dim, bias=False, device=device, dtype=dtype)  # gate | up
        self.c_proj = nn.Linear(cfg.ffn_dim, cfg.n_embd, bias=False, device=device, dtype=dtype)

    def forward(self, x, residual=None):
        return self.c_proj(ops.swiglu(self.c_fc(x)), residual)


class LLaMA3Block(nn.Module):
    kType = "Block"

    def __init__(self, cfg: LLaMA3Config, device=None, dtype=torch.float32):
        super().__init__()
        self.ln_1 = nn.RMSNorm(cfg.n_embd, cfg.norm_eps, device=device, dtype=dtype)
        self.attn = LLaMA3Attention(cfg, device=device, dtype=dtype)
        self.ln_2 = nn.RMSNorm(cfg.n_embd, cfg.norm_eps, device=device, dtype=dtype)
        self.mlp = LLaMA3MLP(cfg, device=device, dtype=dtype)

    def forward(self, x):
        h, x = self.ln_1.fork(x)
        x = self.attn(h, residual=x)
        h, x = self.ln_2.fork(x)
        x = self.mlp(h, residual=x)
        return x


class LLaMA3(nn.Module):
    kType = "LLaMA3"

    def __init__(self, config: LLaMA3Config, device=None, dtype=torch.float32, seed: Optional[int] = 42):
        super().__init__()
        self.config = config
        Cdim = config.n_embd
        self.transformer = nn.ModuleDict({
            "wte": nn.Embedding(config.vocab_size, Cdim, device=device, dtype=dtype),
            "h": nn.Sequential(*[LLaMA3Block(config, device=device, dtype=dtype) for _ in range(config.n_layer)]),
            "ln_f": nn.RMSNorm(Cdim, config.norm_eps, device=device, dtype=dtype),
        })
        self.lm_head = nn.Linear(Cdim, config.vocab_size, bias=False, device=device, dtype=dtype)
        self.reset_parameters(seed)

    def reset_parameters(self, seed: Optional[int] = 42) -> None:
        resid_std = 0.02 / math.sqrt(2 * self.config.n_layer)
        for name, p in self.named_parameters():
            if "ln_" in name:
                init.Ones(p)
            elif name.endswith("c_proj.weight"):
                init.Normal(p, 0.0, resid_std, generator=seed)
            else:
                init.Normal(p, 0.0, 0.02, generator=seed)

    def forward(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None, return_logits: bool = True):
        cfg = self.config
        B, T = idx.shape
        assert T <= cfg.block_size
        tr = self.transformer
        x = ops.embedding(idx, tr["wte"].weight)
        for block in tr["h"]:
            x = block(x)
        x = tr["ln_f"](x)
        w = self.lm_head.weight
        if targets is not None and not return_logits:
            return None, ops.lm_head_loss(x, w, targets, cfg.vocab_size)
        logits = ops.linear(x, w)
        if targets is None:
            return logits
        return logits, ops.cross_entropy(logits, targets, cfg.vocab_size)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self, T: int) -> float:
        n_dense = sum(p.numel() for n, p in self.named_parameters() if "wte" not in n)
        return 6.0 * n_dense + 6.0 * self.config.n_layer * self.config.n_embd * T

    @classmethod
    def FromLLMC(cls, path: str, device=None, dtype=torch.float32) -> "LLaMA3":
        from ..utils import llmc

        return llmc.load_llama3(path, device=device, dtype=dtype)

    def SaveLLMC(self, path: str, bf16: bool = False) -> None:
        from ..utils import llmc

        llmc.save_llama3(self, path, bf16=bf16)

    @classmethod
    def FromPretrained(cls, path_or_name: str, device=None, dtype=torch.float32) -> "LLaMA3":
        """A Hugging Face LLaMA checkpoint directory (opened with ``transformers``, local files only)."""
        from ..utils import hf

        model = hf.from_pretrained(path_or_name, device=device, dtype=dtype)
        assert isinstance(model, cls), f"{path_or_name} is not a LLaMA checkpoint"
        return model
