"""llm.c checkpoint files <-> models (format reader/writer in C++: csrc/core/llmc_io.cc).

GPT-2: header/payload layout of example/gpt2/net.cc:242-374, versions 3 (fp32) and 5 (bf16).
"""
from __future__ import annotations

import torch

from .._lib import C


def load_gpt2(path: str, device=None, dtype=torch.float32):
    from ..models.gpt2 import GPT2, GPT2Config

    hdr, sd = C.llmc_read_gpt2(path, False)
    cfg = GPT2Config(block_size=hdr["block_size"], vocab_size=hdr["vocab_size"], n_layer=hdr["n_layer"],
                     n_head=hdr["n_head"], n_embd=hdr["n_embd"])
    model = GPT2(cfg, device=device, dtype=dtype, seed=None)
    own = model.StateDict()
    with torch.no_grad():
        for name, t in sd.items():
            if name == "lm_head.weight":
                continue  # tied to wte
            dst = own[name]
            if name == "transformer.wte.weight":
                dst[:t.shape[0]].copy_(t.to(dst.dtype))
                dst[t.shape[0]:].zero_()
            else:
                dst.copy_(t.to(dst.dtype))
    return model


def save_gpt2(model, path: str, bf16: bool = False) -> None:
    cfg = model.config
    hdr = {"version": 5 if bf16 else 3, "block_size": cfg.block_size, "vocab_size": cfg.vocab_size,
           "n_layer": cfg.n_layer, "n_head": cfg.n_head, "n_embd": cfg.n_embd,
           "padded_vocab_size": cfg.padded_vocab_size}
    sd = {k: v.detach().float().cpu() for k, v in model.StateDict().items() if k != "lm_head.weight"}
    C.llmc_write_gpt2(path, hdr, sd)


def load_llama3(path: str, device=None, dtype=torch.float32):
    from ..models.llama3 import LLaMA3, LLaMA3Config

    hdr, sd = C.llmc_read_llama3(path)
    cfg = LLaMA3Config(block_size=hdr["max_seq_len"], vocab_size=hdr["vocab_size"], n_layer=hdr["n_layer"],
                       n_head=hdr["n_head"], n_kv_head=hdr["n_kv_head"], n_embd=hdr["n_embd"], ffn_dim=hdr["ffn_dim"],
                       norm_eps=hdr["norm_eps"], rope_theta=hdr["rope_theta"])
    model = LLaMA3(cfg, device=device, dtype=dtype, seed=None)
    own = model.StateDict()
    with torch.no_grad():
        for name, t in sd.items():
            own[name].copy_(t.to(own[name].dtype))
    return model


def save_llama3(model, path: str, bf16: bool = False) -> None:
    cfg = model.config
    hdr = {"version": 5 if bf16 else 3, "max_seq_len": cfg.block_size, "vocab_size": cfg.vocab_size,
           "n_layer": cfg.n_layer, "n_head": cfg.n_head, "n_kv_head": cfg.n_kv_head, "n_embd": cfg.n_embd,
           "ffn_dim": cfg.ffn_dim, "rope_theta": cfg.rope_theta, "norm_eps": cfg.norm_eps}
    sd = {k: v.detach().float().cpu() for k, v in model.StateDict().items()}
    C.llmc_write_llama3(path, hdr, sd)


def map_checkpoint(path: str):
    """Memory-maps an llm.c GPT-2 or LLaMA-3 checkpoint: returns ``(family, header, state_dict)`` whose tensors are
    views into the file (fp32 or bf16, as stored; no copy, pages load when touched).  Used for tensor-parallel
    loading, where each rank slices out its own rows and columns."""
    import struct

    with open(path, "rb") as f:
        magic = struct.unpack("<i", f.read(4))[0]
    if magic == 20240326:
        hdr, sd = C.llmc_map_gpt2(path)
        return "gpt2", hdr, sd
    if magic == 20240803:
        hdr, sd = C.llmc_map_llama3(path)
        return "llama3", hdr, sd
    raise ValueError(f"{path}: unknown checkpoint magic {magic}")
