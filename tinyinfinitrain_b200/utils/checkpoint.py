"""Checkpoint save / resume.

The reference can only load model weights (``GPT2::FromLLMC``, example/gpt2/net.cc:246-377); it
has no save, no optimizer state and no step counter.  Here a checkpoint is a directory:

* ``model.bin``      -- llm.c layout (GPT-2 or LLaMA-3, fp32 or bf16), written by global rank 0; readable by llm.c
  and by the reference's loader (GPT-2 version 3).  In a tensor / pipeline parallel job the ranks of the first
  model replica send their slices to rank 0, which reassembles the full tensors (``gather_full_state_dict``),
* ``optim_rankN.pt`` -- this data-parallel rank's optimizer shard (fp32 master weights, Adam
  moments, step count): with ZeRO-1 every rank owns a different slice,
* ``meta.json``      -- step, world layout, model name.

Resuming restores master weights, moments and the step counter exactly, so the next step after a
resume equals the step an uninterrupted run would have taken.  In a multi-rank job every rank writes
and reads its own ``optim_rankN.pt`` (N = global rank: its tensor / pipeline slice of the model and its
ZeRO shard of that slice); the ZeRO optimizer then rebuilds the full parameter buffers of its
data-parallel group from the master-weight shards.
"""
from __future__ import annotations

import json
import os
from typing import Optional

import torch


def gather_full_state_dict(model, mesh):
    """Collective over the ranks of one model replica (``mesh.mp_group``; every rank of the job may call it, only data-
    parallel replica 0 communicates): returns the unsharded fp32 CPU state dict on global rank 0, None elsewhere."""
    import torch.distributed as dist

    from ..models.tp_models import unshard_state_dict

    if mesh.dp_rank != 0:
        return None
    mine = {k: v.detach().float().cpu() for k, v in model.named_parameters(remove_duplicate=False)}
    payload = (mesh.pp_rank, mesh.tp_rank, mine)
    if mesh.mp_group is None:
        gathered = [payload]
    else:
        gathered = [None] * dist.get_world_size(mesh.mp_group) if mesh.rank == 0 else None
        dist.gather_object(payload, gathered, dst=0, group=mesh.mp_group)
    if mesh.rank != 0:
        return None
    cfg = model.config
    is_llama = model.is_llama
    full = {}
    for stage in range(mesh.pp):
        shards = [sd for (p, t, sd) in sorted((g for g in gathered if g[0] == stage), key=lambda g: g[1])]
        full.update(unshard_state_dict(shards, cfg, cfg.vocab_size if is_llama else cfg.padded_vocab_size))
    if not is_llama:
        head = full.pop("lm_head.weight", None)   # tied to wte in the file format
        if head is not None and not torch.equal(head, full["transformer.wte.weight"]):
            raise RuntimeError("the output projection of the last pipeline stage and the token embedding of the first have "
                               "drifted apart; they are one tied parameter and must be updated with the summed gradient")
    return full


def save_checkpoint(path: str, model, optimizer, step: int, rank: int = 0, world: int = 1, extra: Optional[dict] = None,
                    bf16_weights: bool = False, mesh=None) -> None:
    """``mesh``: the ParallelMesh of a tensor / pipeline / data parallel job (then every rank must call this)."""
    os.makedirs(path, exist_ok=True)

    def publish(name, write):
        # written under a temporary name and renamed: a crash in the middle of a save leaves the previous file intact
        tmp = os.path.join(path, name + ".tmp")
        write(tmp)
        os.replace(tmp, os.path.join(path, name))

    if rank == 0 and hasattr(model, "SaveLLMC"):
        publish("model.bin", lambda p: model.SaveLLMC(p, bf16=bf16_weights))
    elif mesh is not None and hasattr(model, "is_llama"):
        full = gather_full_state_dict(model, mesh)
        if full is not None:
            from .._lib import C

            cfg = model.config
            if model.is_llama:
                hdr = {"version": 5 if bf16_weights else 3, "max_seq_len": cfg.block_size, "vocab_size": cfg.vocab_size,
                       "n_layer": cfg.n_layer, "n_head": cfg.n_head, "n_kv_head": cfg.n_kv_head, "n_embd": cfg.n_embd,
                       "ffn_dim": cfg.ffn_dim, "rope_theta": cfg.rope_theta, "norm_eps": cfg.norm_eps}
                publish("model.bin", lambda p: C.llmc_write_llama3(p, hdr, full))
            else:
                hdr = {"version": 5 if bf16_weights else 3, "block_size": cfg.block_size, "vocab_size": cfg.vocab_size,
                       "n_layer": cfg.n_layer, "n_head": cfg.n_head, "n_embd": cfg.n_embd,
                       "padded_vocab_size": cfg.padded_vocab_size}
                publish("model.bin", lambda p: C.llmc_write_gpt2(p, hdr, full))
    sd = optimizer.state_dict()
    sd["step"] = int(step)
    publish(f"optim_rank{rank}.pt",
            lambda p: torch.save({k: (v.detach().cpu() if torch.is_tensor(v) else v) for k, v in sd.items()}, p))
    if rank == 0:
        meta = {"step": int(step), "world": int(world), "model": type(model).__name__}
        meta.update(extra or {})

        def write_meta(p):
            with open(p, "w") as f:
                json.dump(meta, f)

        publish("meta.json", write_meta)


def load_checkpoint(path: str, model, optimizer, rank: int = 0, world: Optional[int] = None,
                    layout: Optional[dict] = None) -> int:
    """Restores optimizer state (and through the fp32 master weights, the parameters). Returns the step.
    ``world`` and ``layout`` ({"tp", "pp", "dp"}) describe the running job; a checkpoint written by another layout is
    refused, because every ``optim_rankN.pt`` is the shard of one particular rank of one particular layout."""
    with open(os.path.join(path, "meta.json")) as f:
        meta = json.load(f)
    if world is not None and int(meta.get("world", world)) != int(world):
        raise RuntimeError(f"{path}: written by a job of {meta['world']} ranks, this job has {world}")
    for k, v in (layout or {}).items():
        if k in meta and int(meta[k]) != int(v):
            raise RuntimeError(f"{path}: written with {k}={meta[k]}, this job runs {k}={v} (optimizer shards do not line up)")
    sd = torch.load(os.path.join(path, f"optim_rank{rank}.pt"), map_location="cpu")
    if "step" in sd and int(sd["step"]) != int(meta["step"]):
        raise RuntimeError(f"{path}: optimizer shard of rank {rank} is from step {sd['step']}, meta.json says {meta['step']} "
                           "(a save was interrupted between ranks)")
    sd.pop("step", None)
    optimizer.load_state_dict(sd)
    return int(meta["step"])
