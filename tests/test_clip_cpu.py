"""Gradient-norm clipping in the flat optimizers (CPU paths; the CUDA kernels of csrc/kernels/clip.cu follow the same
arithmetic): single-process MixedPrecisionAdam and the ZeRO-1 optimizer over two gloo ranks, both against
torch.nn.utils.clip_grad_norm_ + torch.optim.AdamW on the same gradients."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import tinyinfinitrain_b200 as tit

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_mixed_precision_adam_clips_like_torch():
    torch.manual_seed(0)
    lin, ref = torch.nn.Linear(23, 11), torch.nn.Linear(23, 11)
    ref.load_state_dict(lin.state_dict())
    opt = tit.optim.MixedPrecisionAdam(lin.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=0.5)
    ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    norms = []
    for step in range(4):
        x = torch.randn(6, 23, generator=torch.Generator().manual_seed(step)) * (10.0 if step % 2 == 0 else 0.01)
        opt.zero_grad()
        for p in opt.params:
            p.grad = None
        lin(x).pow(2).mean().backward()          # plain autograd gradients are folded into main_grad by step()
        opt.step()
        ropt.zero_grad()
        ref(x).pow(2).mean().backward()
        norms.append(float(torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.5)))
        ropt.step()
        assert abs(opt.grad_norm() - norms[-1]) < 1e-4 * max(1.0, norms[-1])
    assert max(norms) > 0.5 > min(norms)          # both the clipped and the unclipped case were exercised
    for a, b in zip(lin.parameters(), ref.parameters()):
        assert torch.allclose(a, b, atol=1e-5)


def _worker(rank, world, port, q, kind):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tinyinfinitrain_b200.parallel import AllReduceOptimizer, DistributedOptimizer

        torch.manual_seed(0)
        lin, ref = torch.nn.Linear(37, 19), torch.nn.Linear(37, 19)
        ref.load_state_dict(lin.state_dict())
        cls = DistributedOptimizer if kind == "zero1" else AllReduceOptimizer
        opt = cls(lin.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, max_grad_norm=0.3)
        ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
        ok = True
        for step in range(3):
            scale = 8.0 if step != 1 else 0.01
            xs = [torch.randn(5, 37, generator=torch.Generator().manual_seed(100 * step + r)) * scale for r in range(world)]
            opt.zero_grad()
            for p in opt.params:
                p.grad = None
            lin(xs[rank]).pow(2).mean().backward()
            opt.step()
            ropt.zero_grad()
            sum(ref(x).pow(2).mean() for x in xs).div(world).backward()      # the averaged gradient all ranks agree on
            n = float(torch.nn.utils.clip_grad_norm_(ref.parameters(), 0.3))
            ropt.step()
            ok &= abs(opt.grad_norm() - n) < 1e-4 * max(1.0, n)
        ok &= all(torch.allclose(a, b, atol=1e-5) for a, b in zip(lin.parameters(), ref.parameters()))
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


import pytest  # noqa: E402


@pytest.mark.parametrize("kind", ["zero1", "allreduce"])
def test_data_parallel_optimizers_clip_the_global_norm_over_two_ranks(kind):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29100 + os.getpid() % 300 + (7 if kind == "zero1" else 0)
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, kind)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res == [(0, True), (1, True)], res


def _mp_worker(rank, world, port, q):
    """4 ranks = tensor parallel 2 x data parallel 2.  `w` is sharded over the tensor ranks, `r` is replicated there."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tinyinfinitrain_b200.parallel import AllReduceOptimizer, DistributedOptimizer, init_mesh

        mesh = init_mesh(tp=2, pp=1)                     # rank = dp_rank * 2 + tp_rank
        t, d = mesh.tp_rank, mesh.dp_rank

        def grads(step):
            gw = torch.full((300,), 0.01 * (1 + t) * (1 + 2 * d) * (step + 1))      # differs per tensor and data rank
            gr = torch.full((40,), 0.02 * (1 + d) * (step + 1))                      # same on both tensor ranks
            return gw, gr

        def expected_norm(step):
            tot = 0.0
            for tt in range(2):
                w_avg = sum(0.01 * (1 + tt) * (1 + 2 * dd) * (step + 1) for dd in range(2)) / 2
                tot += 300 * w_avg ** 2
            r_avg = sum(0.02 * (1 + dd) * (step + 1) for dd in range(2)) / 2
            return (tot + 40 * r_avg ** 2) ** 0.5

        ok = True
        for cls in (DistributedOptimizer, AllReduceOptimizer):
            torch.manual_seed(0)
            w, r = torch.nn.Parameter(torch.randn(300)), torch.nn.Parameter(torch.randn(40))
            r._sp_grad_sync = True
            opt = cls([w, r], lr=1e-2, group=mesh.dp_group, max_grad_norm=0.05, mp_group=mesh.mp_group, tp_world=2)
            assert opt.flat.params[0] is r and opt.flat.n_replicated == 128        # replicated parameters come first
            for step in range(2):
                opt.zero_grad()
                w.grad, r.grad = grads(step)
                before = w.detach().clone()
                opt.step()
                n = expected_norm(step)
                ok &= abs(opt.grad_norm() - n) < 1e-5 * max(1.0, n)
                ok &= bool((w.detach() - before).abs().max() > 0)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_global_norm_counts_tensor_parallel_replicas_once():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29180 + os.getpid() % 100
    procs = [ctx.Process(target=_mp_worker, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=30)
    assert res == [(r, True) for r in range(4)], res
