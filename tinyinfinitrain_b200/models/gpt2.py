"""GPT-2 (llm.c / TinyInfiniTrain layout) on the fused sm_100a operators.

Reference: example/gpt2/net.h:13-78 and net.cc:46-221.  Layer and parameter
names match, so ``StateDict()`` keys are the reference's
(``transformer.wte.weight``, ``transformer.h.0.attn.c_attn.weight``, ...,
``lm_head.weight``).  Per block the GPU path launches: LayerNorm, QKV GEMM
(+bias), fused causal attention reading q/k/v in place from the QKV buffer,
output-projection GEMM (+bias +residual), LayerNorm, MLP GEMM (+bias +GELU),
MLP GEMM (+bias +residual) -- 7 kernels where the reference runs about 40.

Deliberate differences from the reference model:
* the embedding/lm_head matrix is one tied parameter, padded to a multiple of
  128 rows (50257 -> 50304) for tensor-core tiles; pad rows are zero and their
  logits are masked out of the loss;
* ``lm_head`` has no bias (the reference's GPT2Linear always adds one,
  net.cc:32-33,167, which llm.c checkpoints do not contain).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch

from .. import nn, ops
from ..nn import init


@dataclass
class GPT2Config:
    block_size: int = 1024
    vocab_size: int = 50257
    n_layer: int = 12
    n_head: int = 12
    n_embd: int = 768
    padded_vocab_size: Optional[int] = None

    def __post_init__(self):
        if self.padded_vocab_size is None:
            self.padded_vocab_size = (self.vocab_size + 127) // 128 * 128


GPT2_PRESETS = {
    "gpt2": GPT2Config(n_layer=12, n_head=12, n_embd=768),
    "gpt2-medium": GPT2Config(n_layer=24, n_head=16, n_embd=1024),
    "gpt2-large": GPT2Config(n_layer=36, n_head=20, n_embd=1280),
    "gpt2-xl": GPT2Config(n_layer=48, n_head=25, n_embd=1600),
}


class NewGELU(nn.Module):
    kType = "NewGELU"

    def forward(self, x):
        return ops.gelu(x)


class CausalSelfAttention(nn.Module):
    kType = "CausalSelfAttention"

    def __init__(self, config: GPT2Config, device=None, dtype=torch.float32):
        super().__init__()
        assert config.n_embd % config.n_head == 0
        self.n_head, self.n_embd = config.n_head, config.n_embd
        self.c_attn = nn.Linear(config.n_embd, 3 * config.n_embd, device=device, dtype=dtype)
        self.c_proj = nn.Linear(config.n_embd, config.n_embd, device=device, dtype=dtype)

    def forward(self, x, residual=None):
        B, T, Cdim = x.shape
        H, hd = self.n_head, Cdim // self.n_head
        qkv = self.c_attn(x)  # [B, T, 3C]; q, k, v are read in place by the attention kernel
        y = ops.causal_attention_qkv(qkv, H).reshape(B, T, Cdim)
        return self.c_proj(y, residual)


class MLP(nn.Module):
    kType = "MLP"

    def __init__(self, config: GPT2Config, device=None, dtype=torch.float32):
        super().__init__()
        self.c_fc = nn.Linear(config.n_embd, 4 * config.n_embd, device=device, dtype=dtype)
        self.gelu = NewGELU()
        self.c_proj = nn.Linear(4 * config.n_embd, config.n_embd, device=device, dtype=dtype)

    def forward(self, x, residual=None):
        return ops.mlp_gelu(x, self.c_fc.weight, self.c_fc.bias, self.c_proj.weight, self.c_proj.bias, residual)


class Block(nn.Module):
    kType = "Block"

    def __init__(self, config: GPT2Config, device=None, dtype=torch.float32):
        super().__init__()
        self.ln_1 = nn.LayerNorm(config.n_embd, device=device, dtype=dtype)
        self.attn = CausalSelfAttention(config, device=device, dtype=dtype)
        self.ln_2 = nn.LayerNorm(config.n_embd, device=device, dtype=dtype)
        self.mlp = MLP(config, device=device, dtype=dtype)

    def forward(self, x):
        h, x = self.ln_1.fork(x)
        x = self.attn(h, residual=x)
        h, x = self.ln_2.fork(x)
        x = self.mlp(h, residual=x)
        return x


class _LMHead(nn.Module):
    kType = "Linear"

    def __init__(self, weight: torch.nn.Parameter):
        super().__init__()
        self.weight = weight


class GPT2(nn.Module):
    kType = "GPT2"

    def __init__(self, config: GPT2Config, device=None, dtype=torch.float32, seed: Optional[int] = 42):
        super().__init__()
        self.config = config
        Vp, Cdim = config.padded_vocab_size, config.n_embd
        wte = nn.Embedding(Vp, Cdim, device=device, dtype=dtype)
        wpe = nn.Embedding(config.block_size, Cdim, device=device, dtype=dtype)
        self.transformer = nn.ModuleDict({
            "wte": wte,
            "wpe": wpe,
            "h": nn.Sequential(*[Block(config, device=device, dtype=dtype) for _ in range(config.n_layer)]),
            "ln_f": nn.LayerNorm(Cdim, device=device, dtype=dtype),
        })
        self.lm_head = _LMHead(wte.weight)  # tied: one parameter under two names
        self.reset_parameters(seed)

    # ---- initialisation (example/gpt2/net.cc:175-188) -----------------------------------
    def reset_parameters(self, seed: Optional[int] = 42) -> None:
        """N(0, 0.02) weights, residual projections N(0, 0.02/sqrt(2 L)), zero biases, LN 1/0.
        Every tensor is drawn from the start of the ``seed`` stream, as in the reference
        where the seeded generator is copied per call (nn/init.h:12-13, init.cc:29)."""
        cfg = self.config
        resid_std = 0.02 / math.sqrt(2 * cfg.n_layer)
        for name, p in self.named_parameters():
            if name.endswith("ln_1.weight") or name.endswith("ln_2.weight") or name.endswith("ln_f.weight"):
                init.Ones(p)
            elif name.endswith(".bias"):
                init.Zeros(p)
            elif name.endswith("c_proj.weight"):
                init.Normal(p, 0.0, resid_std, generator=seed)
            else:
                init.Normal(p, 0.0, 0.02, generator=seed)
        with torch.no_grad():
            self.transformer["wte"].weight[cfg.vocab_size:].zero_()

    # ---- forward ------------------------------------------------------------------------------
    def forward(self, idx: torch.Tensor, targets: Optional[torch.Tensor] = None, return_logits: bool = True):
        """``idx``: int64 [B, T].  Without ``targets`` returns logits [B, T, vocab_size].
        With ``targets`` returns ``(logits, loss)``; ``return_logits=False`` takes the fused
        projection + loss path that never materialises a separate gradient tensor and
        returns ``(None, loss)``."""
        cfg = self.config
        B, T = idx.shape
        assert T <= cfg.block_size, f"sequence of length {T} exceeds block size {cfg.block_size}"
        tr = self.transformer
        x = ops.embedding(idx, tr["wte"].weight, tr["wpe"].weight)
        for block in tr["h"]:
            x = block(x)
        x = tr["ln_f"](x)
        w = self.lm_head.weight
        if targets is not None and not return_logits:
            return None, ops.lm_head_loss(x, w, targets, cfg.vocab_size)
        logits = ops.linear(x, w)
        loss = None
        if targets is not None:
            loss = ops.cross_entropy(logits, targets, cfg.vocab_size)
        return (logits[..., :cfg.vocab_size], loss) if targets is not None else logits[..., :cfg.vocab_size]

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def flops_per_token(self, T: int) -> float:
        """Training FLOPs per token: 6 N for the dense layers plus causal attention."""
        cfg = self.config
        n_dense = sum(p.numel() for n, p in self.named_parameters() if "wpe" not in n)
        return 6.0 * n_dense + 6.0 * cfg.n_layer * cfg.n_embd * T

    # ---- llm.c checkpoints (example/gpt2/net.cc:228-377) ------------------------------------------
    @classmethod
    def FromLLMC(cls, path: str, device=None, dtype=torch.float32) -> "GPT2":
        from ..utils import llmc

        return llmc.load_gpt2(path, device=device, dtype=dtype)

    def SaveLLMC(self, path: str, bf16: bool = False) -> None:
        from ..utils import llmc

        llmc.save_gpt2(self, path, bf16=bf16)

    @classmethod
    def FromPretrained(cls, path_or_name: str, device=None, dtype=torch.float32) -> "GPT2":
        """A Hugging Face GPT-2 checkpoint directory or cached model name, opened with ``transformers`` without
        network access (the reference's FromPretrained aborts: example/gpt2/net.cc:223-226)."""
        from ..utils import hf

        model = hf.from_pretrained(path_or_name, device=device, dtype=dtype)
        assert isinstance(model, cls), f"{path_or_name} is not a GPT-2 checkpoint"
        return model
