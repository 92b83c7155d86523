"""The reference's end-to-end logits check (test/example/test_gpt2.cc), restated: blob format, sampling
rule, and the 11-step SGD protocol.  The full 124M run needs the llm.c starter pack (directory named by
TITB200_LLMC_DATA holding gpt2_124M.bin, tiny_shakespeare_train.bin and gpt2_logits_reference.bin)."""
import os
import struct

import pytest
import torch

from tinyinfinitrain_b200.models import GPT2, GPT2Config
from tinyinfinitrain_b200.utils import logits_check as lc


def test_blob_roundtrip_and_layout(tmp_path):
    t = torch.randn(2, 5, 7)
    p = str(tmp_path / "blob.bin")
    lc.write_logits_blob(p, t)
    raw = open(p, "rb").read()
    assert struct.unpack("<Q", raw[:8])[0] == 3
    assert struct.unpack("<3q", raw[8:32]) == (2, 5, 7)
    assert len(raw) == 32 + 4 * 70
    assert torch.equal(lc.read_logits_blob(p), t)


def test_sampling_rule_and_tolerance(tmp_path):
    t = torch.zeros(2, 64, 50)
    p = str(tmp_path / "ref.bin")
    lc.write_logits_blob(p, t)
    idx = lc.sample_indices(t.numel())
    assert len(idx) == 100 and idx[0] == 0 and idx[1] == t.numel() // 100 and idx[99] == 99 * t.numel() // 100
    cur = t.clone().reshape(-1)
    cur[idx[7] + 1] = 5.0             # not a sampled position: ignored, like the reference
    ok, worst = lc.validate_logits(cur.view_as(t), p)
    assert ok and worst == 0.0
    cur[idx[7]] = 2e-3                # sampled position beyond the 1e-3 tolerance
    ok, worst = lc.validate_logits(cur.view_as(t), p)
    assert not ok and abs(worst - 2e-3) < 1e-9
    assert lc.validate_logits(torch.zeros(2, 64, 49), p)[0] is False   # shape mismatch fails


class _Tokens(torch.utils.data.Dataset):
    def __init__(self, n, T, vocab):
        g = torch.Generator().manual_seed(3)
        self.tok = torch.randint(0, vocab, (n * T + 1,), generator=g)
        self.T = T

    def __len__(self):
        return (len(self.tok) - 1) // self.T

    def __getitem__(self, i):
        s = i * self.T
        return self.tok[s:s + self.T], self.tok[s + 1:s + self.T + 1]


def test_protocol_is_deterministic_and_learns(tmp_path):
    cfg = GPT2Config(block_size=16, vocab_size=97, n_layer=2, n_head=2, n_embd=32)
    ds = _Tokens(8, 16, 97)
    runs = []
    for _ in range(2):
        model = GPT2(cfg, seed=42)
        runs.append(lc.run_reference_protocol(model, ds, "cpu", batch_size=2, total_batch_size=64, num_iteration=3,
                                              learning_rate=1e-2))
    assert runs[0].shape == (2, 16, 97)
    p = str(tmp_path / "ref.bin")
    lc.write_logits_blob(p, runs[0])
    ok, worst = lc.validate_logits(runs[1], p)
    assert ok and worst == 0.0
    fresh = GPT2(cfg, seed=42)
    x = torch.stack([ds[2][0], ds[3][0]])       # the last micro-step's batch
    assert (fresh(x) - runs[0]).abs().max() > 1e-4  # the SGD steps changed the logits


@pytest.mark.skipif(not os.environ.get("TITB200_LLMC_DATA"), reason="llm.c starter pack not present")
def test_gpt2_124m_logits_match_reference_blob():
    ok, worst = lc.run_from_starter_pack(os.environ["TITB200_LLMC_DATA"], "cuda" if torch.cuda.is_available() else "cpu")
    assert ok, f"worst sampled |diff| = {worst}"
