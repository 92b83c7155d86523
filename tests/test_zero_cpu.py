"""ZeRO-1 sharding logic on CPU ranks (gloo, world_size 2): sharded Adam == full Adam on summed grads."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tinyinfinitrain_b200.parallel import DistributedOptimizer

        torch.manual_seed(0)
        lin = torch.nn.Linear(37, 19)
        ref = torch.nn.Linear(37, 19)
        ref.load_state_dict(lin.state_dict())
        opt = DistributedOptimizer(lin.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
        ropt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
        for step in range(3):
            xs = [torch.randn(5, 37, generator=torch.Generator().manual_seed(100 * step + r)) for r in range(world)]
            opt.zero_grad()
            for p in opt.params:  # emulate the wgrad kernels: write main_grad directly
                p.grad = None
            loss = lin(xs[rank]).pow(2).mean()
            loss.backward()
            for p in opt.params:
                p.main_grad.copy_(p.grad)
                p._fresh_grad = False
                p.grad = None  # a leftover .grad would be folded into main_grad a second time by step()
            opt.step()
            ropt.zero_grad()
            sum(ref(x).pow(2).mean() for x in xs).div(world).backward()
            ropt.step()
        ok = all(torch.allclose(a, b, atol=1e-5) for a, b in zip(lin.parameters(), ref.parameters()))
        q.put((rank, ok))
    finally:
        dist.destroy_process_group()


def test_zero1_two_cpu_ranks():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=30)
    assert all(ok for _, ok in res), res
