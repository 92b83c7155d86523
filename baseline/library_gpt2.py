"""Library baseline for the headline benchmark: the same GPT-2 architecture, loss and optimizer built
from stock PyTorch pieces only -- cuBLAS GEMMs (``nn.Linear``), ``scaled_dot_product_attention``,
``F.layer_norm``, ``F.gelu(approximate="tanh")``, ``F.cross_entropy``, fused ``torch.optim.AdamW`` and
NCCL through ``DistributedDataParallel``.  None of this repository's kernels, models or engine is on
this path; it is the stand-in for "the reference algorithm through libraries" (the reference itself
cannot be built, see bench.py) and the number the hand-written path has to beat.

Mixed precision follows the usual library recipe: fp32 parameters, bf16 autocast.
"""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class Block(nn.Module):
    def __init__(self, C: int, H: int):
        super().__init__()
        self.H = H
        self.ln_1, self.ln_2 = nn.LayerNorm(C), nn.LayerNorm(C)
        self.c_attn, self.c_proj = nn.Linear(C, 3 * C), nn.Linear(C, C)
        self.c_fc, self.mlp_proj = nn.Linear(C, 4 * C), nn.Linear(4 * C, C)

    def forward(self, x):
        B, T, C = x.shape
        q, k, v = self.c_attn(self.ln_1(x)).split(C, dim=2)
        q, k, v = (t.view(B, T, self.H, C // self.H).transpose(1, 2) for t in (q, k, v))
        y = F.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(B, T, C)
        x = x + self.c_proj(y)
        return x + self.mlp_proj(F.gelu(self.c_fc(self.ln_2(x)), approximate="tanh"))


class LibraryGPT2(nn.Module):
    def __init__(self, vocab_size=50257, padded_vocab_size=50304, block_size=1024, n_layer=12, n_head=12, n_embd=768):
        super().__init__()
        self.vocab_size = vocab_size
        self.wte, self.wpe = nn.Embedding(padded_vocab_size, n_embd), nn.Embedding(block_size, n_embd)
        self.h = nn.ModuleList(Block(n_embd, n_head) for _ in range(n_layer))
        self.ln_f = nn.LayerNorm(n_embd)
        torch.manual_seed(42)
        for name, p in self.named_parameters():
            if p.dim() == 2:
                std = 0.02 / math.sqrt(2 * n_layer) if name.endswith("c_proj.weight") or name.endswith("mlp_proj.weight") else 0.02
                nn.init.normal_(p, 0.0, std)

    @torch.no_grad()
    def load_named(self, sd) -> None:
        """Copies weights given under the GPT-2 state-dict names of the reference (``transformer.h.0.attn.c_attn.weight``
        ...), so that this model and the hand-written one can start a comparison from identical parameters."""
        def name_of(k: str) -> str:
            k = k.replace("transformer.", "")
            k = k.replace("attn.c_attn", "c_attn").replace("attn.c_proj", "c_proj")
            return k.replace("mlp.c_fc", "c_fc").replace("mlp.c_proj", "mlp_proj")

        own = dict(self.named_parameters())
        for k, v in sd.items():
            if k == "lm_head.weight":
                continue
            own[name_of(k)].copy_(v.to(own[name_of(k)].dtype))

    def forward(self, idx, targets):
        T = idx.shape[1]
        x = self.wte(idx) + self.wpe(torch.arange(T, device=idx.device))
        for b in self.h:
            x = b(x)
        logits = F.linear(self.ln_f(x), self.wte.weight)[..., :self.vocab_size]
        return F.cross_entropy(logits.reshape(-1, self.vocab_size).float(), targets.reshape(-1))


class LibraryTrainStep:
    """forward + backward + AdamW step with bf16 autocast; ``__call__`` copies pinned host tokens in and
    returns the loss tensor (device), mirroring the call the hand-written arm times end to end."""

    def __init__(self, model, B, T, dev, world):
        self.dev = dev
        self.model = model
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP

            self.model = DDP(model, device_ids=[dev.index] if dev.type == "cuda" else None, gradient_as_bucket_view=True)
        self.opt = torch.optim.AdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1,
                                     fused=dev.type == "cuda")
        self.idx = torch.zeros(B, T, dtype=torch.long, device=dev)
        self.tgt = torch.zeros(B, T, dtype=torch.long, device=dev)
        self.loss = None

    def run_device(self):
        self.opt.zero_grad(set_to_none=True)
        with torch.autocast(self.dev.type, dtype=torch.bfloat16):
            loss = self.model(self.idx, self.tgt)
        loss.backward()
        self.opt.step()
        self.loss = loss.detach()
        return self.loss

    def __call__(self, host_idx, host_tgt):
        self.idx.copy_(host_idx, non_blocking=True)
        self.tgt.copy_(host_tgt, non_blocking=True)
        return self.run_device()
