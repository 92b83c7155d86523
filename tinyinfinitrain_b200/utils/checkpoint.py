"""Checkpoint save / resume.

The reference can only load model weights (``GPT2::FromLLMC``, example/gpt2/net.cc:246-377); it
has no save, no optimizer state and no step counter.  Here a checkpoint is a directory:

* ``model.bin``      -- llm.c layout (GPT-2 or LLaMA-3, fp32 or bf16), written by rank 0 of each
  model-parallel layout; readable by llm.c and by the reference's loader (GPT-2 version 3),
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


def save_checkpoint(path: str, model, optimizer, step: int, rank: int = 0, world: int = 1, extra: Optional[dict] = None,
                    bf16_weights: bool = False) -> None:
    os.makedirs(path, exist_ok=True)

    def publish(name, write):
        # written under a temporary name and renamed: a crash in the middle of a save leaves the previous file intact
        tmp = os.path.join(path, name + ".tmp")
        write(tmp)
        os.replace(tmp, os.path.join(path, name))

    if rank == 0 and hasattr(model, "SaveLLMC"):
        publish("model.bin", lambda p: model.SaveLLMC(p, bf16=bf16_weights))
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


def load_checkpoint(path: str, model, optimizer, rank: int = 0) -> int:
    """Restores optimizer state (and through the fp32 master weights, the parameters). Returns the step."""
    with open(os.path.join(path, "meta.json")) as f:
        meta = json.load(f)
    sd = torch.load(os.path.join(path, f"optim_rank{rank}.pt"), map_location="cpu")
    if "step" in sd and int(sd["step"]) != int(meta["step"]):
        raise RuntimeError(f"{path}: optimizer shard of rank {rank} is from step {sd['step']}, meta.json says {meta['step']} "
                           "(a save was interrupted between ranks)")
    sd.pop("step", None)
    optimizer.load_state_dict(sd)
    return int(meta["step"])
