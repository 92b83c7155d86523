"""The reference's end-to-end acceptance check, restated (test/example/test_gpt2.cc:26-101 and :149-227).

Blob layout: ``uint64 ndims; int64 dims[ndims]; float32 data[prod(dims)]`` (little endian).  The check
compares 100 evenly spaced elements (index ``i * numel // 100``) with an absolute tolerance of 1e-3.

Protocol that produces the tensor under test: GPT-2 124M from the llm.c file, batch 2 x 64 tokens from the
start of the TinyShakespeare training file, 2 micro-steps per optimizer step (256 tokens), plain SGD with
lr 1e-4, 11 optimizer steps.  Every step restarts the loader, so all steps see the same two batches; the
loss of each micro-step is back-propagated undivided; the logits of the last micro-step are compared.
"""
from __future__ import annotations

import os
import struct
from typing import Sequence, Tuple

import numpy as np
import torch

SAMPLE_COUNT = 100
DEFAULT_TOLERANCE = 1e-3


def write_logits_blob(path: str, logits: torch.Tensor) -> None:
    t = logits.detach().to("cpu", torch.float32).contiguous()
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", t.dim()))
        f.write(struct.pack(f"<{t.dim()}q", *t.shape))
        f.write(t.numpy().tobytes())


def read_logits_blob(path: str) -> torch.Tensor:
    with open(path, "rb") as f:
        (nd,) = struct.unpack("<Q", f.read(8))
        if nd == 0 or nd > 8:
            raise ValueError(f"{path}: implausible number of dimensions {nd}")
        dims = struct.unpack(f"<{nd}q", f.read(8 * nd))
        n = int(np.prod(dims))
        data = np.fromfile(f, dtype="<f4", count=n)
    if data.size != n:
        raise ValueError(f"{path}: expected {n} floats, file holds {data.size}")
    return torch.from_numpy(data.reshape(dims).copy())


def sample_indices(numel: int, count: int = SAMPLE_COUNT) -> Sequence[int]:
    return [i * numel // count for i in range(count)]


def validate_logits(logits: torch.Tensor, reference_path: str, tolerance: float = DEFAULT_TOLERANCE) -> Tuple[bool, float]:
    """Returns (passed, worst absolute difference over the sampled positions)."""
    ref = read_logits_blob(reference_path)
    if tuple(ref.shape) != tuple(logits.shape):
        return False, float("inf")
    cur = logits.detach().to("cpu", torch.float32).reshape(-1)
    idx = torch.tensor(sample_indices(ref.numel()), dtype=torch.long)
    worst = (cur[idx] - ref.reshape(-1)[idx]).abs().max().item()
    return worst <= tolerance, worst


def run_reference_protocol(model, dataset, device, batch_size: int = 2, total_batch_size: int = 256,
                           num_iteration: int = 10, learning_rate: float = 1e-4) -> torch.Tensor:
    """Runs the 11 SGD steps of the reference test and returns the last micro-step's logits [B, T, vocab]."""
    from .. import nn, optim
    from ..data import DataLoader

    seq_len = dataset[0][0].shape[-1]
    accum = total_batch_size // (batch_size * seq_len)
    opt = optim.SGD(model.parameters(), learning_rate)
    loss_fn = nn.CrossEntropyLoss()
    logits = None
    for _ in range(num_iteration + 1):
        it = iter(DataLoader(dataset, batch_size))
        opt.zero_grad()
        for _ in range(accum):
            x, y = next(it)
            x, y = x.to(device), y.to(device)
            logits = model(x)
            loss = loss_fn(logits.reshape(-1, logits.shape[-1]), y.reshape(-1))
            loss.backward()
        opt.step()
    return logits[..., :model.config.vocab_size].detach()


def run_from_starter_pack(data_dir: str, device: str = "cpu"):
    """Loads ``gpt2_124M.bin`` and ``tiny_shakespeare_train.bin`` from an llm.c starter pack directory, runs
    the protocol and validates against ``gpt2_logits_reference.bin`` in the same directory."""
    from ..data import TinyShakespeareDataset
    from .llmc import load_gpt2

    model = load_gpt2(os.path.join(data_dir, "gpt2_124M.bin"), device=device, dtype=torch.float32)
    tokens = os.path.join(data_dir, "tinyshakespeare", "tiny_shakespeare_train.bin")
    if not os.path.exists(tokens):
        tokens = os.path.join(data_dir, "tiny_shakespeare_train.bin")
    logits = run_reference_protocol(model, TinyShakespeareDataset(tokens, 64), device)
    return validate_logits(logits, os.path.join(data_dir, "gpt2_logits_reference.bin"))
