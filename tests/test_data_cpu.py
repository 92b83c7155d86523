"""Data layer in C++ (csrc/core/data.cc): llm.c token files, dataset windows, loader batching and rank sharding,
tokenizer table, and llm.c's sampling generator.  Semantics from the reference's example/common/
tiny_shakespeare_dataset.cc:27-40,74-82, tokenizer.cc:14-69 and src/dataloader.cc:16-56."""
import pytest
import torch

from tinyinfinitrain_b200 import data
from tinyinfinitrain_b200._lib import C


def _xorshift_u32(state):
    mask = (1 << 64) - 1
    state ^= state >> 12
    state = (state ^ (state << 25)) & mask
    state ^= state >> 27
    return ((state * 0x2545F4914F6CDD1D) & mask) >> 32, state


@pytest.mark.parametrize("magic,dtype_max", [(20240520, 65535), (20240801, 200000)])
def test_token_file_roundtrip_and_windows(tmp_path, magic, dtype_max):
    toks = torch.randint(0, dtype_max, (1000,), generator=torch.Generator().manual_seed(1))
    path = str(tmp_path / "toks.bin")
    C.llmc_write_tokens(path, toks, magic)
    back, m = C.llmc_read_tokens(path)
    assert m == magic and back.dtype == torch.int64 and torch.equal(back, toks)
    raw = open(path, "rb").read()
    assert len(raw) == 1024 + toks.numel() * (2 if magic == 20240520 else 4)     # 256-int header + payload

    ds = data.TinyShakespeareDataset(path, 64)
    assert ds.NumTokens() == 1000 and len(ds) == (1000 - 1) // 64 and ds.SequenceLength() == 64
    assert ds.is_uint32() == (magic == 20240801)
    x, y = ds[3]
    assert x.dtype == torch.int64 and torch.equal(x, toks[192:256]) and torch.equal(y, toks[193:257])   # y = x shifted by one
    with pytest.raises((RuntimeError, IndexError)):
        ds[len(ds)]


def test_token_file_rejects_other_magic(tmp_path):
    p = tmp_path / "bad.bin"
    p.write_bytes(b"\x01" * 2048)
    with pytest.raises(RuntimeError):
        data.TinyShakespeareDataset(str(p), 8)


def test_loader_batches_and_rank_sharding(tmp_path):
    toks = torch.arange(0, 16 * 10 + 1)
    path = str(tmp_path / "t.bin")
    C.llmc_write_tokens(path, toks, 20240520)
    ds = data.TinyShakespeareDataset(path, 16)           # 10 samples
    dl = data.DataLoader(ds, 4)
    assert len(dl) == 3                                  # 4 + 4 + 2: the last batch is short, as in the reference
    batches = list(dl)
    assert [tuple(b[0].shape) for b in batches] == [(4, 16), (4, 16), (2, 16)]
    assert torch.equal(batches[1][0][0], toks[64:80]) and torch.equal(batches[1][1][0], toks[65:81])
    # two data-parallel ranks take interleaved batches and together cover every sample once
    seen = []
    for r in range(2):
        part = list(data.DataLoader(ds, 4, rank=r, world=2))
        assert len(part) == (2 if r == 0 else 1)
        seen += [int(b[0][i, 0]) for b in part for i in range(b[0].shape[0])]
    assert sorted(seen) == [16 * i for i in range(10)]


def test_synthetic_dataset_is_seeded_and_in_range():
    a, b = data.SyntheticDataset(7, 50257, 32, 5), data.SyntheticDataset(7, 50257, 32, 5)
    c = data.SyntheticDataset(8, 50257, 32, 5)
    assert len(a) == 5
    xa, ya = a[2]
    assert torch.equal(xa, b[2][0]) and not torch.equal(xa, c[2][0])
    assert torch.equal(xa[1:], ya[:-1]) and int(xa.min()) >= 0 and int(xa.max()) < 50257


@pytest.mark.parametrize("magic,eot,prompt", [(20240328, 50256, [464, 3616, 286, 1204, 318]),
                                              (20240801, 128001, [791, 7438, 315, 2324, 374])])
def test_tokenizer_table_eot_and_prompt(tmp_path, magic, eot, prompt):
    table = [bytes([65 + i % 26]) * (1 + i % 3) for i in range(300)]
    table[7] = "é".encode()                              # multi-byte entry
    path = str(tmp_path / "tok.bin")
    C.write_tokenizer(path, table, magic, eot)
    tk = data.Tokenizer(path)
    assert tk.vocab_size == 300 and tk.GetEndToken() == eot
    assert tk.Decode(0) == "A" and tk.Decode(2) == "CCC" and tk.Decode(7) == "é"
    assert tk._t.Prompt() == prompt and tk._t.Magic() == magic


def test_llmc_random_generator_and_sampling():
    state = 1337
    for _ in range(5):
        exp, exp_state = _xorshift_u32(state)
        got, got_state = C.random_u32(state)
        assert got == exp and got_state == exp_state
        f, f_state = C.random_f32(state)
        assert f == pytest.approx((exp >> 8) / 16777216.0, abs=0) and f_state == exp_state and 0.0 <= f < 1.0
        state = exp_state
    probs = torch.tensor([0.1, 0.2, 0.3, 0.4])
    assert [C.sample_mult(probs, c) for c in (0.0, 0.0999, 0.1, 0.29, 0.3, 0.61, 0.999)] == [0, 0, 1, 1, 2, 3, 3]
    assert C.sample_mult(torch.tensor([0.25, 0.25]), 0.9) == 1      # rounding guard: falls back to the last index


def test_generate_text_walks_the_window(tmp_path):
    table = [f"<{i}>".encode() for i in range(50300)]
    path = str(tmp_path / "tok.bin")
    C.write_tokenizer(path, table, 20240328, 50256)
    tk = data.Tokenizer(path)

    class Peaked(torch.nn.Module):       # always predicts token (previous token + 1) with probability 1
        def forward(self, x):
            logits = torch.full((*x.shape, 50300), -1e4)
            logits.scatter_(2, ((x + 1) % 50300).unsqueeze(-1), 1e4)
            return logits

    text = tk.GenerateText(Peaked(), 2, 16, 9, "cpu")
    assert text == "The meaning of life is" + "<319><320><321><322>"       # 4 tokens after the 5-token prompt (318 + 1 ...)


def test_drop_last_serves_full_batches_and_equal_counts_per_rank():
    """11 samples, batch 2, 2 ranks: 5 full batches -> 2 per rank (the 5th full batch and the short one are dropped);
    without drop_last rank 0 gets 3 batches, rank 1 gets 3 and its last one is short."""
    from tinyinfinitrain_b200 import data

    ds = data.SyntheticDataset(1, 100, 8, 11)
    for rank in range(2):
        dl = data.DataLoader(ds, 2, rank=rank, world=2, drop_last=True)
        assert len(dl) == 2
        assert all(dl.batch(i)[0].shape == (2, 8) for i in range(len(dl)))
    loose = [data.DataLoader(ds, 2, rank=r, world=2) for r in range(2)]
    assert [len(d) for d in loose] == [3, 3] and loose[1].batch(2)[0].shape == (1, 8)
