"""1F1B pipeline on 2 CPU ranks (gloo): schedule order, and loss/gradients against one process."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def test_schedule_order_and_partition():
    from tinyinfinitrain_b200.parallel.pp import one_f_one_b_order, partition_layers

    assert [list(r) for r in partition_layers(5, 2)] == [[0, 1, 2], [3, 4]]
    assert one_f_one_b_order(0, 2, 4) == [("F", 0), ("F", 1), ("B", 0), ("F", 2), ("B", 1), ("F", 3), ("B", 2), ("B", 3)]
    assert one_f_one_b_order(1, 2, 4) == [("F", 0), ("B", 0), ("F", 1), ("B", 1), ("F", 2), ("B", 2), ("F", 3), ("B", 3)]
    for s in range(4):  # never more than P - s activations alive
        alive = peak = 0
        for kind, _ in one_f_one_b_order(s, 4, 8):
            alive += 1 if kind == "F" else -1
            peak = max(peak, alive)
        assert peak <= 4 - s


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tinyinfinitrain_b200.models import GPT2, GPT2Config
        from tinyinfinitrain_b200.models.tp_models import TPTransformer
        from tinyinfinitrain_b200.parallel import mesh as pm
        from tinyinfinitrain_b200.parallel.pp import PipelineStage, partition_layers
        from tinyinfinitrain_b200.parallel.tp import TPComm

        m = pm.init_mesh(tp=1, pp=world)
        cfg = GPT2Config(block_size=32, vocab_size=250, n_layer=4, n_head=2, n_embd=32)
        full = GPT2(cfg)
        layers = partition_layers(cfg.n_layer, world)[m.pp_rank]
        stage = TPTransformer(cfg, TPComm(None), layers=layers, first=m.is_first_stage, last=m.is_last_stage)
        sd = dict(full.StateDict())
        stage.load_full_state_dict(sd)
        B, T, nm = 2, 16, 4
        g = torch.Generator().manual_seed(11)
        idx = [torch.randint(0, cfg.vocab_size, (B, T), generator=g) for _ in range(nm)]
        tgt = [torch.roll(x, -1, 1) for x in idx]

        def fwd(x_in, i):
            if m.is_first_stage:
                return stage(idx[i])
            return stage(x_in, tgt[i] if m.is_last_stage else None, B=B, T=T)

        ps = PipelineStage(fwd, m.pp_rank, world, None if m.is_first_stage else m.prev_stage_rank(),
                           None if m.is_last_stage else m.next_stage_rank(), (B * T, cfg.n_embd), torch.float32, "cpu")
        ps.trace = []
        loss = ps.run(nm)
        trace = list(ps.trace)
        ref_loss = sum(full(idx[i], tgt[i])[1] for i in range(nm)) / nm
        ref_loss.backward()
        ref = {k: v.grad for k, v in full.StateDict().items() if v.grad is not None}
        worst = 0.0
        for name, p in stage.named_parameters():
            if p.grad is None or name not in ref:
                continue
            if name in ("transformer.wte.weight", "lm_head.weight"):
                continue  # tied in the reference model, split across stages here
            r = ref[name]
            worst = max(worst, (p.grad[:r.shape[0]] - r).abs().max().item())
        ok = worst < 1e-4 and (loss is None or abs(loss.item() - ref_loss.item()) < 1e-4)
        q.put((rank, ok, worst, None if loss is None else loss.item(), ref_loss.item(), trace))
    finally:
        dist.destroy_process_group()


def test_1f1b_two_stages_match_single_process():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + os.getpid() % 90
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(r[1] for r in res), res


def _check_trace(trace, stage, P, nm):
    """What the overlap needs from the schedule: the compute order is 1F1B, a batch that only sends is never waited
    for before the last forward / backward has been launched, and in the warm-up and cool-down phases the receive of
    the next micro-batch is posted before the current one is computed."""
    from tinyinfinitrain_b200.parallel.pp import one_f_one_b_order

    compute = [e for e in trace if e[0] in ("F", "B")]
    assert compute == one_f_one_b_order(stage, P, nm), compute
    last_compute = max(i for i, e in enumerate(trace) if e[0] in ("F", "B"))
    send_waits = [i for i, e in enumerate(trace) if e == ("wait", "s")]
    assert all(i > last_compute for i in send_waits), trace
    n_send_only = sum(1 for e in trace if e == ("issue", "s"))
    assert len(send_waits) == n_send_only                                  # every deferred handle is drained once
    warm = min(P - stage - 1, nm)
    if stage > 0 and warm >= 1:
        # two receives are in flight before the first forward starts: its own input and the next one
        first_f = trace.index(("F", 0))
        assert sum(1 for e in trace[:first_f] if e == ("issue", "r")) == 2, trace[:first_f]
    if stage < P - 1 and warm >= 2:
        first_cooldown_b = trace.index(("B", nm - warm))
        tail = trace[first_cooldown_b - 3:first_cooldown_b]
        assert tail.count(("issue", "r")) >= 1, trace


def test_schedule_defers_send_waits_and_prefetches_receives():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + os.getpid() % 90
    P, nm = 4, 4           # the worker runs 4 micro-batches
    procs = [ctx.Process(target=_worker, args=(r, P, port, q)) for r in range(P)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(r[1] for r in res), [r[:5] for r in res]
    for r in res:
        _check_trace(r[5], r[0], P, nm)
