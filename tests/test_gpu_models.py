"""Model-level GPU checks against the CPU fp32 oracle."""
import pytest
import torch

import tinyinfinitrain_b200 as tit
from tinyinfinitrain_b200._lib import C

pytestmark = pytest.mark.gpu


def test_llama3_tiny_matches_cpu_oracle_and_trains():
    from tinyinfinitrain_b200.models import LLaMA3, LLaMA3Config

    cfg = LLaMA3Config(block_size=256, vocab_size=1000, n_layer=2, n_head=4, n_kv_head=2, n_embd=256, ffn_dim=512)
    cpu = LLaMA3(cfg)
    gpu = LLaMA3(cfg, device="cuda", dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(3)
    idx = torch.randint(0, 1000, (2, 200), generator=g)
    tgt = torch.roll(idx, -1, 1)
    _, l_cpu = cpu(idx, tgt)
    _, l_gpu = gpu(idx.cuda(), tgt.cuda(), return_logits=False)
    assert abs(l_cpu.item() - l_gpu.item()) < 3e-2
    opt = tit.optim.MixedPrecisionAdam(gpu.parameters(), lr=1e-3)
    first = last = None
    for _ in range(8):
        opt.zero_grad()
        _, loss = gpu(idx.cuda(), tgt.cuda(), return_logits=False)
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
        last = loss.item()
    torch.cuda.synchronize()
    assert C.status_read(True) == 0
    assert last < first - 0.5, (first, last)


def test_train_step_graph_matches_eager():
    from tinyinfinitrain_b200.models import GPT2, GPT2Config
    from tinyinfinitrain_b200.utils import TrainStep

    cfg = GPT2Config(block_size=128, vocab_size=1000, n_layer=2, n_head=4, n_embd=256)
    g = torch.Generator().manual_seed(5)
    idx = torch.randint(0, 1000, (4, 128), generator=g).pin_memory()
    tgt = torch.roll(idx, -1, 1).pin_memory()
    out = []
    for use_graph in (False, True):
        model = GPT2(cfg, device="cuda", dtype=torch.bfloat16)
        opt = tit.optim.MixedPrecisionAdam(model.parameters(), lr=1e-3)
        step = TrainStep(model, opt, 4, 128, "cuda", use_graph=use_graph)
        step.idx.copy_(idx); step.tgt.copy_(tgt)
        step.prepare(eager_warmup=1)
        losses = []
        for _ in range(5):
            hl = step(idx, tgt)
            torch.cuda.synchronize()
            losses.append(float(hl))
        out.append(losses)
    assert all(abs(a - b) < 5e-2 for a, b in zip(*out)), out
    assert out[1][-1] < out[1][0]
