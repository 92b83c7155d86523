"""Tensor + sequence parallel GPT-2 and LLaMA-3.

Same layer names as the single-GPU models; every rank holds its slice of each weight:
``c_attn`` (heads), ``c_fc`` (hidden units) and ``wte`` / ``lm_head`` (vocabulary rows) are
split by output rows, the two ``c_proj`` by input columns; norm weights, biases of the row
parallel layers and ``wpe`` are replicated.  Activations between blocks are token shards
``[B*T/tp, C]``.  ``shard_state_dict`` cuts a full model's tensors into one rank's slices.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import nn, ops
from ..nn import init
from ..parallel import tp as tpl
from .gpt2 import GPT2Config
from .llama3 import LLaMA3Config


def head_range(n: int, tp: int, rank: int):
    """[first, last) of the heads rank ``rank`` owns; the first ``n % tp`` ranks take one extra head
    (GPT-2 XL has 25 heads, which two ranks split 13 / 12)."""
    base, rem = divmod(n, tp)
    first = rank * base + min(rank, rem)
    return first, first + base + (1 if rank < rem else 0)


def _qkv_rows(n_head: int, n_kv_head: int, hd: int, tp: int, rank: int):
    """Row indices of a fused [q | k | v] projection that belong to one tensor-parallel rank."""
    q0, q1 = head_range(n_head, tp, rank)
    k0, k1 = head_range(n_kv_head, tp, rank)
    q = torch.arange(q0 * hd, q1 * hd)
    k = n_head * hd + torch.arange(k0 * hd, k1 * hd)
    v = (n_head + n_kv_head) * hd + torch.arange(k0 * hd, k1 * hd)
    return torch.cat([q, k, v])


def shard_state_dict(sd: Dict[str, torch.Tensor], cfg, tp: int, rank: int, vocab_padded: int = 0) -> Dict[str, torch.Tensor]:
    """Slices a full GPT-2 / LLaMA-3 state dict for tensor-parallel rank ``rank`` of ``tp``.  ``vocab_padded`` is
    the row count the vocabulary-sharded tensors are padded to (zero rows) before they are split."""
    is_llama = isinstance(cfg, LLaMA3Config)
    n_kv = cfg.n_kv_head if is_llama else cfg.n_head
    hd = cfg.n_embd // cfg.n_head
    out = {}
    for name, t in sd.items():
        if name.endswith("attn.c_attn.weight") or name.endswith("attn.c_attn.bias"):
            out[name] = t[_qkv_rows(cfg.n_head, n_kv, hd, tp, rank)]
        elif name.endswith("mlp.c_fc.weight") or name.endswith("mlp.c_fc.bias"):
            if is_llama:  # rows are [gate | up]
                F = t.shape[0] // 2
                f = F // tp
                out[name] = torch.cat([t[rank * f:(rank + 1) * f], t[F + rank * f:F + (rank + 1) * f]])
            else:
                n = t.shape[0] // tp
                out[name] = t[rank * n:(rank + 1) * n]
        elif name.endswith("attn.c_proj.weight"):
            q0, q1 = head_range(cfg.n_head, tp, rank)
            out[name] = t[:, q0 * hd:q1 * hd]
        elif name.endswith("c_proj.weight"):
            n = t.shape[1] // tp
            out[name] = t[:, rank * n:(rank + 1) * n]
        elif name in ("transformer.wte.weight", "lm_head.weight"):
            rows = max(vocab_padded, t.shape[0]) if vocab_padded else t.shape[0]
            n = rows // tp
            lo, hi = rank * n, (rank + 1) * n
            part = t[min(lo, t.shape[0]):min(hi, t.shape[0])]
            if part.shape[0] < n:  # this rank's range reaches into the zero padding
                part = torch.cat([part, torch.zeros(n - part.shape[0], t.shape[1], dtype=t.dtype)])
            out[name] = part
        else:
            out[name] = t
    return {k: v.contiguous() for k, v in out.items()}


def unshard_state_dict(shards, cfg, vocab_rows: int) -> Dict[str, torch.Tensor]:
    """Inverse of ``shard_state_dict``: ``shards[r]`` holds tensor-parallel rank r's tensors (same names on every
    rank); returns the unsharded tensors.  ``vocab_rows`` is the row count the vocabulary tensors are cut back to
    (the padding rows that were added for an even split carry no information)."""
    tp = len(shards)
    is_llama = isinstance(cfg, LLaMA3Config)
    n_kv = cfg.n_kv_head if is_llama else cfg.n_head
    hd = cfg.n_embd // cfg.n_head
    out = {}
    for name in shards[0]:
        parts = [sh[name] for sh in shards]
        if name.endswith("attn.c_attn.weight") or name.endswith("attn.c_attn.bias"):
            q, k, v = [], [], []
            for r, t in enumerate(parts):
                q0, q1 = head_range(cfg.n_head, tp, r)
                k0, k1 = head_range(n_kv, tp, r)
                nq, nk = (q1 - q0) * hd, (k1 - k0) * hd
                q.append(t[:nq]); k.append(t[nq:nq + nk]); v.append(t[nq + nk:nq + 2 * nk])
            out[name] = torch.cat(q + k + v)
        elif name.endswith("mlp.c_fc.weight") or name.endswith("mlp.c_fc.bias"):
            if is_llama:
                f = parts[0].shape[0] // 2
                out[name] = torch.cat([t[:f] for t in parts] + [t[f:] for t in parts])
            else:
                out[name] = torch.cat(parts)
        elif name.endswith("c_proj.weight"):
            out[name] = torch.cat(parts, dim=1)
        elif name in ("transformer.wte.weight", "lm_head.weight"):
            out[name] = torch.cat(parts)[:vocab_rows]
        else:
            out[name] = parts[0]
    return {k: v.contiguous() for k, v in out.items()}


class TPAttention(nn.Module):
    kType = "CausalSelfAttention"

    def __init__(self, n_embd, n_head, n_kv_head, comm, bias, rope_theta=None, device=None, dtype=torch.float32):
        super().__init__()
        self.hd = n_embd // n_head
        q0, q1 = head_range(n_head, comm.world, comm.rank)
        k0, k1 = head_range(n_kv_head, comm.world, comm.rank)
        self.hq, self.hk = q1 - q0, k1 - k0
        assert self.hk > 0 and self.hq % self.hk == 0, "every rank needs whole groups of query heads per kv head"
        self.rope_theta = rope_theta
        self.c_attn = tpl.ColumnParallelLinear(n_embd, (n_head + 2 * n_kv_head) * self.hd, comm, bias, device, dtype,
                                               out_local=(self.hq + 2 * self.hk) * self.hd)
        self.c_proj = tpl.RowParallelLinear(n_embd, n_embd, comm, bias, device, dtype, in_local=self.hq * self.hd)

    def forward(self, x_s, B: int, T: int, residual_s=None):
        qkv = self.c_attn(x_s).view(B, T, -1)
        if self.rope_theta is not None:
            qkv = ops.rope_qkv(qkv, self.hq + self.hk, self.hd, 0, self.rope_theta)
        y = ops.causal_attention_qkv(qkv, self.hq, self.hk)
        return self.c_proj(y.reshape(B * T, self.hq * self.hd), residual_s)


class TPGPT2MLP(nn.Module):
    kType = "MLP"

    def __init__(self, n_embd, comm, device=None, dtype=torch.float32):
        super().__init__()
        self.comm = comm
        self.c_fc = tpl.ColumnParallelLinear(n_embd, 4 * n_embd, comm, True, device, dtype)
        self.c_proj = tpl.RowParallelLinear(4 * n_embd, n_embd, comm, True, device, dtype)

    def forward(self, x_s, residual_s=None):
        return tpl._TPMLPGeluFn.apply(x_s, self.c_fc.weight, self.c_fc.bias, self.c_proj.weight, self.c_proj.bias,
                                      residual_s, self.comm)


class TPLLaMAMLP(nn.Module):
    kType = "MLP"

    def __init__(self, n_embd, ffn_dim, comm, device=None, dtype=torch.float32):
        super().__init__()
        self.c_fc = tpl.ColumnParallelLinear(n_embd, 2 * ffn_dim, comm, False, device, dtype)  # local [gate | up]
        self.c_proj = tpl.RowParallelLinear(ffn_dim, n_embd, comm, False, device, dtype)

    def forward(self, x_s, residual_s=None):
        return self.c_proj(ops.swiglu(self.c_fc(x_s)), residual_s)


class TPBlock(nn.Module):
    kType = "Block"

    def __init__(self, cfg, comm, device=None, dtype=torch.float32):
        super().__init__()
        self.comm = comm
        llama = isinstance(cfg, LLaMA3Config)
        if llama:
            self.ln_1 = nn.RMSNorm(cfg.n_embd, cfg.norm_eps, device=device, dtype=dtype)
            self.ln_2 = nn.RMSNorm(cfg.n_embd, cfg.norm_eps, device=device, dtype=dtype)
            self.attn = TPAttention(cfg.n_embd, cfg.n_head, cfg.n_kv_head, comm, False, cfg.rope_theta, device, dtype)
            self.mlp = TPLLaMAMLP(cfg.n_embd, cfg.ffn_dim, comm, device, dtype)
        else:
            self.ln_1 = nn.LayerNorm(cfg.n_embd, device=device, dtype=dtype)
            self.ln_2 = nn.LayerNorm(cfg.n_embd, device=device, dtype=dtype)
            self.attn = TPAttention(cfg.n_embd, cfg.n_head, cfg.n_head, comm, True, None, device, dtype)
            self.mlp = TPGPT2MLP(cfg.n_embd, comm, device, dtype)
        for ln in (self.ln_1, self.ln_2):
            for p in ln.parameters():
                tpl._mark_sp(p)

    def forward(self, x_s, B: int, T: int):
        # the norms write straight into the input slot of the all-gather -> GEMM kernel that consumes them
        h_s, x_s = self.ln_1.fork(x_s, out=self.comm.ag_input(x_s))
        x_s = self.attn(h_s, B, T, residual_s=x_s)
        h_s, x_s = self.ln_2.fork(x_s, out=self.comm.ag_input(x_s))
        x_s = self.mlp(h_s, residual_s=x_s)
        return x_s


class TPTransformer(nn.Module):
    """GPT-2 or LLaMA-3 (chosen by the config type) on one tensor-parallel group.

    ``layers`` restricts the module to a contiguous range of blocks (a pipeline stage);
    ``first``/``last`` say whether the stage owns the embedding / the final norm + lm_head.
    """

    kType = "TPTransformer"

    def __init__(self, cfg, comm: tpl.TPComm, device=None, dtype=torch.float32, seed: Optional[int] = 42,
                 layers: Optional[range] = None, first: bool = True, last: bool = True, exact_init_limit: int = 1 << 26):
        super().__init__()
        self.config, self.comm = cfg, comm
        self.is_llama = isinstance(cfg, LLaMA3Config)
        self.first, self.last = first, last
        self.layer_ids = list(layers) if layers is not None else list(range(cfg.n_layer))
        Cdim = cfg.n_embd
        vp = cfg.vocab_size if self.is_llama else cfg.padded_vocab_size
        gran = 128 * comm.world
        self.vocab_padded = (vp + gran - 1) // gran * gran
        mods = {}
        if first:
            mods["wte"] = tpl.VocabParallelEmbedding(self.vocab_padded, Cdim, comm, device, dtype)
            if not self.is_llama:
                mods["wpe"] = nn.Embedding(cfg.block_size, Cdim, device=device, dtype=dtype)
                tpl._mark_sp(mods["wpe"].weight)
        mods["h"] = nn.ModuleDict({str(i): TPBlock(cfg, comm, device, dtype) for i in self.layer_ids})
        if last:
            mods["ln_f"] = (nn.RMSNorm(Cdim, cfg.norm_eps, device=device, dtype=dtype) if self.is_llama
                            else nn.LayerNorm(Cdim, device=device, dtype=dtype))
            for p in mods["ln_f"].parameters():
                tpl._mark_sp(p)
        self.transformer = nn.ModuleDict(mods)
        if last:
            if self.is_llama or not first:
                self.lm_head = nn.Module()
                self.lm_head.weight = torch.nn.Parameter(
                    torch.empty(self.vocab_padded // comm.world, Cdim, device=device, dtype=dtype))
            else:
                self.lm_head = nn.Module()
                self.lm_head.weight = self.transformer["wte"].weight  # tied (GPT-2, single stage)
        self.reset_parameters(seed, exact_init_limit)

    def full_shape(self, name: str, p: torch.Tensor):
        """Shape of the unsharded tensor that parameter ``name`` is a slice of."""
        cfg = self.config
        hd = cfg.n_embd // cfg.n_head
        n_kv = cfg.n_kv_head if self.is_llama else cfg.n_head
        if name.endswith("attn.c_attn.weight"):
            return ((cfg.n_head + 2 * n_kv) * hd, cfg.n_embd)
        if name.endswith("mlp.c_fc.weight"):
            return ((2 * cfg.ffn_dim if self.is_llama else 4 * cfg.n_embd), cfg.n_embd)
        if name.endswith("attn.c_proj.weight"):
            return (cfg.n_embd, cfg.n_embd)
        if name.endswith("mlp.c_proj.weight"):
            return (cfg.n_embd, cfg.ffn_dim if self.is_llama else 4 * cfg.n_embd)
        if name in ("transformer.wte.weight", "lm_head.weight"):
            return (cfg.vocab_size if self.is_llama else cfg.padded_vocab_size, cfg.n_embd)
        return tuple(p.shape)

    def reset_parameters(self, seed: Optional[int], exact_limit: int = 1 << 26) -> None:
        """Same distributions as the single-GPU models.  A sharded parameter whose unsharded tensor has at most
        ``exact_limit`` elements is drawn in full on the host from the start of the ``seed`` stream and this rank's
        slice is copied, which reproduces the single-GPU model of the same seed exactly.  Larger tensors (the big
        LLaMA matrices) are drawn on the device from a generator seeded with (seed, tensor-parallel rank, parameter
        index), so that no two shards and no two layers repeat each other.  Replicated parameters are identical on
        every rank of the group in both cases."""
        cfg, comm = self.config, self.comm
        resid_std = 0.02 / math.sqrt(2 * cfg.n_layer)
        own = {}
        for name, p in self.named_parameters(remove_duplicate=False):
            if id(p) not in {id(q) for q in own.values()}:
                own[name] = p
        for index, (name, p) in enumerate(own.items()):
            if "ln_" in name and name.endswith("weight"):
                init.Ones(p)
                continue
            if name.endswith(".bias"):
                init.Zeros(p)
                continue
            std = resid_std if name.endswith("c_proj.weight") else 0.02
            full = self.full_shape(name, p)
            if full == tuple(p.shape):                 # replicated (or a group of one rank)
                init.Normal(p, 0.0, std, generator=seed)
            elif math.prod(full) <= exact_limit:
                t = init.Normal(torch.empty(full, dtype=torch.float32), 0.0, std, generator=seed)
                if not self.is_llama and name in ("transformer.wte.weight", "lm_head.weight"):
                    t[cfg.vocab_size:].zero_()         # padding rows of the GPT-2 vocabulary
                mine = shard_state_dict({name: t}, cfg, comm.world, comm.rank, vocab_padded=self.vocab_padded)[name]
                with torch.no_grad():
                    p.copy_(mine.to(device=p.device, dtype=p.dtype))
            else:
                g = torch.Generator(device=p.device)
                g.manual_seed(((0 if seed is None else int(seed)) * 1000003 + comm.rank) * 1000003 + index)
                with torch.no_grad():
                    p.copy_((torch.randn(p.shape, generator=g, device=p.device, dtype=torch.float32) * std).to(p.dtype))

    def load_full_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        """Loads this rank's slices from a full (unsharded) state dict of the single-GPU model.  The tensors may
        be memory-mapped views of a checkpoint file (``utils.llmc.map_checkpoint``): slicing happens before any
        copy, so a rank only reads its own rows and columns of the file."""
        mine = shard_state_dict(sd, self.config, self.comm.world, self.comm.rank, vocab_padded=self.vocab_padded)
        own = dict(self.named_parameters(remove_duplicate=False))
        with torch.no_grad():
            for name, p in own.items():
                if name in mine:
                    p.copy_(mine[name].to(device=p.device, dtype=p.dtype))

    def embed(self, idx):
        B, T = idx.shape
        x_s = self.transformer["wte"](idx)
        if not self.is_llama:
            Ms = x_s.shape[0]
            rows = torch.arange(self.comm.rank * Ms, (self.comm.rank + 1) * Ms, device=idx.device)
            x_s = x_s + ops.embedding(rows % T, self.transformer["wpe"].weight)
        return x_s

    def forward(self, idx_or_x, targets=None, B: Optional[int] = None, T: Optional[int] = None):
        """First stage: ``idx`` int64 [B, T]; later stages: the previous stage's token shard plus B, T.
        Last stage with ``targets`` returns the loss, otherwise the token shard is returned."""
        self.comm.new_step()
        if self.first:
            B, T = idx_or_x.shape
            x_s = self.embed(idx_or_x)
        else:
            x_s = idx_or_x
        for i in self.layer_ids:
            x_s = self.transformer["h"][str(i)](x_s, B, T)
        if not self.last:
            return x_s
        x_s = self.transformer["ln_f"](x_s)
        if targets is None:
            return x_s
        return tpl.vocab_parallel_lm_head_loss(x_s, self.lm_head.weight, targets, self.config.vocab_size, self.comm)
