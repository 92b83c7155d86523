"""Tensor + sequence parallel models on 2 CPU ranks (gloo) against the single-process model."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q, which):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tinyinfinitrain_b200.models import GPT2, GPT2Config, LLaMA3, LLaMA3Config
        from tinyinfinitrain_b200.models.tp_models import TPTransformer, shard_state_dict
        from tinyinfinitrain_b200.parallel import mesh as pm
        from tinyinfinitrain_b200.parallel.tp import TPComm, sync_sequence_parallel_grads

        m = pm.init_mesh(tp=world, pp=1)
        comm = TPComm(m.tp_group)
        if which == "gpt2":
            cfg, cls = GPT2Config(block_size=32, vocab_size=250, n_layer=2, n_head=4, n_embd=32), GPT2
        elif which == "gpt2_uneven_heads":   # 3 heads over 2 ranks: 2 + 1 (GPT-2 XL splits 25 heads 13 + 12)
            cfg, cls = GPT2Config(block_size=32, vocab_size=250, n_layer=2, n_head=3, n_embd=48), GPT2
        else:
            cfg, cls = LLaMA3Config(block_size=32, vocab_size=256, n_layer=2, n_head=4, n_kv_head=2, n_embd=64,
                                    ffn_dim=96), LLaMA3
        full = cls(cfg)
        tp = TPTransformer(cfg, comm)
        # same seed => every rank's parameters are exactly its slices of the single-process model's
        want = shard_state_dict({k: v.detach() for k, v in full.StateDict().items()}, cfg, world, rank,
                                vocab_padded=tp.vocab_padded)
        seeded_ok = True
        for name, p in tp.named_parameters(remove_duplicate=False):
            if name in want:
                seeded_ok = seeded_ok and torch.equal(p.detach(), want[name].to(p.dtype))
        # tensors too large to draw in full on the host: shards differ between ranks and between layers,
        # replicated parameters stay identical across the group
        tp.reset_parameters(42, exact_limit=0)
        mine = {n: p.detach().clone() for n, p in tp.named_parameters()}
        k0, k1 = "transformer.h.0.mlp.c_fc.weight", "transformer.h.1.mlp.c_fc.weight"
        seeded_ok = seeded_ok and not torch.equal(mine[k0], mine[k1])
        gathered = [torch.empty_like(mine[k0]) for _ in range(world)]
        dist.all_gather(gathered, mine[k0])
        seeded_ok = seeded_ok and not torch.equal(gathered[0], gathered[1])
        rep = "transformer.h.0.ln_1.weight" if which == "llama3" else "transformer.wpe.weight"
        gathered = [torch.empty_like(mine[rep]) for _ in range(world)]
        dist.all_gather(gathered, mine[rep])
        seeded_ok = seeded_ok and torch.equal(gathered[0], gathered[1])
        tp.load_full_state_dict(full.StateDict())
        g = torch.Generator().manual_seed(7)
        idx = torch.randint(0, cfg.vocab_size, (2, 16), generator=g)
        tgt = torch.roll(idx, -1, 1)
        _, l0 = full(idx, tgt)
        l1 = tp(idx, tgt)
        l0.backward()
        l1.backward()
        sync_sequence_parallel_grads(tp.parameters(), comm)
        ok = abs(l0.item() - l1.item()) < 1e-4
        ref = shard_state_dict({k: v.grad for k, v in full.StateDict().items() if v.grad is not None}, cfg, world, rank)
        worst = 0.0
        for name, p in tp.named_parameters():
            if name in ref and p.grad is not None:
                r = ref[name]
                worst = max(worst, (p.grad[:r.shape[0]] - r).abs().max().item())
        q.put((rank, ok and worst < 1e-4 and seeded_ok, l0.item(), l1.item(), worst, seeded_ok))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("which", ["gpt2", "gpt2_uneven_heads", "llama3"])
def test_tp2_matches_single_process(which):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29900 + (os.getpid() + hash(which)) % 90
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, which)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(r[1] for r in res), res


@pytest.mark.parametrize("which,tp", [("gpt2", 2), ("gpt2", 3), ("llama3", 2), ("llama3", 4)])
def test_unshard_inverts_shard(which, tp):
    sys.path.insert(0, ROOT)
    from tinyinfinitrain_b200.models import GPT2, GPT2Config, LLaMA3, LLaMA3Config
    from tinyinfinitrain_b200.models.tp_models import shard_state_dict, unshard_state_dict

    if which == "gpt2":
        cfg, cls = GPT2Config(block_size=16, vocab_size=250, n_layer=1, n_head=6, n_embd=48), GPT2
        rows = cfg.padded_vocab_size
    else:
        cfg, cls = LLaMA3Config(block_size=16, vocab_size=256, n_layer=1, n_head=8, n_kv_head=4, n_embd=64, ffn_dim=96), LLaMA3
        rows = cfg.vocab_size
    full = {k: v.detach() for k, v in cls(cfg).StateDict().items()}
    padded = (rows + 128 * tp - 1) // (128 * tp) * (128 * tp)
    shards = [shard_state_dict(full, cfg, tp, r, vocab_padded=padded) for r in range(tp)]
    back = unshard_state_dict(shards, cfg, rows)
    assert set(back) == set(full)
    for k in full:
        assert torch.equal(back[k], full[k]), k
