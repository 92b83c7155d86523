"""Save / resume: the step after a resume equals the step an uninterrupted run takes."""
import pytest
import torch

import tinyinfinitrain_b200 as tit
from tinyinfinitrain_b200.models import GPT2, GPT2Config
from tinyinfinitrain_b200.utils import load_checkpoint, save_checkpoint


def _run(tmp_path, device, dtype, resume_at=None):
    cfg = GPT2Config(block_size=32, vocab_size=130, n_layer=2, n_head=2, n_embd=64)
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, 130, (2, 32), generator=g).to(device)
    tgt = torch.roll(idx, -1, 1)
    model = GPT2(cfg, device=device, dtype=dtype)
    opt = tit.optim.MixedPrecisionAdam(model.parameters(), lr=1e-2)
    losses = []
    for step in range(6):
        if resume_at is not None and step == resume_at:
            # throw everything away and come back from the checkpoint written at this step
            model = GPT2(cfg, device=device, dtype=dtype, seed=7)
            opt = tit.optim.MixedPrecisionAdam(model.parameters(), lr=1e-2)
            assert load_checkpoint(str(tmp_path / "ck"), model, opt) == step
        opt.zero_grad()
        _, loss = model(idx, tgt, return_logits=False)
        loss.backward()
        opt.step()
        losses.append(loss.item())
        if resume_at is None and step == 2:
            save_checkpoint(str(tmp_path / "ck"), model, opt, step + 1)
    return losses


def test_resume_is_exact_cpu(tmp_path):
    a = _run(tmp_path, "cpu", torch.float32)
    b = _run(tmp_path, "cpu", torch.float32, resume_at=3)
    assert a[3:] == b[3:], (a, b)
    m = GPT2.FromLLMC(str(tmp_path / "ck" / "model.bin"))      # weights file is a valid llm.c checkpoint
    assert m.config.n_layer == 2


def test_mapped_checkpoint_views_equal_the_reader_and_shard_lazily(tmp_path):
    """Memory-mapped llm.c checkpoints: same tensors as the copying reader (fp32 and bf16 payloads, GPT-2 and
    LLaMA-3), and tensor-parallel slices taken from the views equal slices of the fully loaded state dict."""
    import torch

    from tinyinfinitrain_b200._lib import C
    from tinyinfinitrain_b200.models import GPT2, GPT2Config, LLaMA3, LLaMA3Config
    from tinyinfinitrain_b200.models.tp_models import shard_state_dict
    from tinyinfinitrain_b200.utils import llmc

    g = GPT2(GPT2Config(block_size=16, vocab_size=97, n_layer=2, n_head=4, n_embd=32), seed=42)
    l = LLaMA3(LLaMA3Config(block_size=16, vocab_size=128, n_layer=2, n_head=4, n_kv_head=2, n_embd=32, ffn_dim=64), seed=42)
    for bf16 in (False, True):
        pg, pl = str(tmp_path / f"g{int(bf16)}.bin"), str(tmp_path / f"l{int(bf16)}.bin")
        llmc.save_gpt2(g, pg, bf16=bf16)
        llmc.save_llama3(l, pl, bf16=bf16)
        for path, family, reader, cfg in ((pg, "gpt2", lambda p: C.llmc_read_gpt2(p, True), g.config),
                                          (pl, "llama3", C.llmc_read_llama3, l.config)):
            fam, hdr, mapped = llmc.map_checkpoint(path)
            _, full = reader(path)
            assert fam == family and set(mapped) == set(full)
            for k in full:
                assert mapped[k].dtype == (torch.bfloat16 if bf16 else torch.float32)
                assert torch.equal(mapped[k].float(), full[k]), k
            for rank in range(2):
                a = shard_state_dict(mapped, cfg, 2, rank, vocab_padded=256)
                b = shard_state_dict(full, cfg, 2, rank, vocab_padded=256)
                for k in a:
                    assert a[k].shape == b[k].shape and torch.equal(a[k].float(), b[k]), k
                assert a["transformer.wte.weight"].shape[0] == 128
            del mapped   # tensors sliced from the views stay valid: the mapping lives while any of them does
            assert float(a["transformer.ln_f.weight"].float().sum()) == float(b["transformer.ln_f.weight"].sum())
    with pytest.raises(ValueError):
        bad = tmp_path / "bad.bin"
        bad.write_bytes(b"\\x00" * 2048)
        llmc.map_checkpoint(str(bad))
