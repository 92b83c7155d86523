"""Data layer: datasets, data loader and tokenizer (implemented in C++: csrc/core/data.cc).

Reference API: ``Dataset`` (infini_train/include/dataset.h:10-16), ``DataLoader``
(dataloader.h:11-42), ``TinyShakespeareDataset`` and ``Tokenizer`` (example/common).
"""
from __future__ import annotations

from typing import Iterator, Optional, Tuple

import torch

from .._lib import C


class Dataset:
    """Abstract dataset: ``ds[i] -> (x, y)`` and ``Size()``."""

    def __getitem__(self, idx: int) -> Tuple[torch.Tensor, torch.Tensor]:
        raise NotImplementedError

    def Size(self) -> int:
        raise NotImplementedError

    def __len__(self) -> int:
        return self.Size()


def TinyShakespeareDataset(filepath: str, sequence_length: int):
    """llm.c token file (.bin, uint16 GPT-2 or uint32 LLaMA-3 tokens) cut into windows of
    ``sequence_length`` tokens; ``ds[i]`` returns the window and its one-token-shifted target."""
    return C.TinyShakespeareDataset(filepath, sequence_length)


def SyntheticDataset(seed: int, vocab_size: int, sequence_length: int, num_samples: int):
    """Uniform random token ids in [0, vocab_size) from std::mt19937(seed)."""
    return C.SyntheticDataset(seed, vocab_size, sequence_length, num_samples)


class DataLoader:
    """Sequential batches of ``batch_size`` samples as two int64 ``[batch, seq]`` tensors.

    Batches are assembled by the C++ loader (directly into pinned memory when ``pin_memory``);
    ``rank``/``world`` give every data-parallel rank a disjoint, interleaved set of batches.
    Python ``Dataset`` subclasses are batched with ``torch.stack`` instead.
    """

    def __init__(self, dataset, batch_size: int, pin_memory: bool = False, rank: int = 0, world: int = 1,
                 drop_last: bool = False):
        """``drop_last``: only full batches, and the same number of them on every rank (what a multi-rank job with
        static shapes needs; without it the last batch may be short and ranks may differ by one batch)."""
        self.dataset, self.batch_size, self.rank, self.world = dataset, batch_size, rank, world
        self.drop_last = drop_last
        self._native = C.DataLoader(dataset, batch_size, pin_memory, rank, world, drop_last) \
            if isinstance(dataset, C.Dataset) else None
        self.pin_memory = pin_memory

    def __len__(self) -> int:
        if self._native is not None:
            return len(self._native)
        if self.drop_last:
            return (len(self.dataset) // self.batch_size) // self.world
        total = (len(self.dataset) + self.batch_size - 1) // self.batch_size
        return max(0, (total - self.rank + self.world - 1) // self.world)

    def batch(self, i: int):
        if self._native is not None:
            return self._native.Batch(i)
        g = self.rank + i * self.world
        items = [self.dataset[j] for j in range(g * self.batch_size, min(len(self.dataset), (g + 1) * self.batch_size))]
        x, y = torch.stack([a for a, _ in items]), torch.stack([b for _, b in items])
        return (x.pin_memory(), y.pin_memory()) if self.pin_memory else (x, y)

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        for i in range(len(self)):
            yield self.batch(i)


class Tokenizer:
    """llm.c tokenizer table: ``Decode`` and sampling-based ``GenerateText``
    (example/common/tokenizer.cc:71-116)."""

    def __init__(self, filepath: str):
        self._t = C.Tokenizer(filepath)

    def Decode(self, token_id: int) -> str:
        return self._t.Decode(int(token_id)).decode("utf-8", errors="replace")

    def GetEndToken(self) -> int:
        return self._t.GetEndToken()

    @property
    def vocab_size(self) -> int:
        return self._t.VocabSize()

    @torch.no_grad()
    def GenerateText(self, model, batch_size: int, sequence_length: int, text_length: int, device,
                     rng_state: int = 1337, stream=None) -> str:
        """Fills a [batch, seq] window with the end token, writes the prompt "The meaning of life is",
        then samples one token at a time from row 0 with llm.c's xorshift generator (no KV cache,
        the whole window is re-run per token, as in the reference)."""
        eot = self.GetEndToken()
        x = torch.full((batch_size, sequence_length), eot, dtype=torch.int64)
        prompt = self._t.Prompt()
        x[0, :len(prompt)] = torch.tensor(prompt, dtype=torch.int64)
        out = "The meaning of life is"
        state = rng_state
        limit = min(text_length, sequence_length)
        for t in range(len(prompt), limit):
            logits = model(x.to(device))
            if isinstance(logits, (tuple, list)):
                logits = logits[0]
            probs = torch.softmax(logits[0, t - 1].float().cpu(), dim=-1)
            coin, state = C.random_f32(state)
            tok = C.sample_mult(probs, coin)
            x[0, t] = tok
            out += self.Decode(tok)
        if stream is not None:
            stream.write(out + "\n")
        return out
