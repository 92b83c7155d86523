"""Save / resume: the step after a resume equals the step an uninterrupted run takes."""
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
