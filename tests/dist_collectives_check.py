"""Multi-GPU check of the standalone symmetric-memory collectives (run under torch.distributed.run, one rank per GPU):
all-reduce (fp32 and bf16, sum and mean, whole buffer and an aligned sub-range) and all-gather against NCCL, eager and
captured in a CUDA graph, and plain data parallelism with the symmetric all-reduce against the NCCL one."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from tinyinfinitrain_b200._lib import C  # noqa: E402
from tinyinfinitrain_b200.parallel import AllReduceOptimizer  # noqa: E402
from tinyinfinitrain_b200.parallel.collectives import SymmCollective  # noqa: E402


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    # TITB_TEST_DEVICE=cpu: the same script over gloo ranks and the CPU fallbacks of the same classes -- a dry run of
    # this script's own logic (references, tolerances, call signatures) that needs no GPU
    on_gpu = os.environ.get("TITB_TEST_DEVICE", "cuda") != "cpu"
    if on_gpu:
        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    sync = torch.cuda.synchronize if on_gpu else (lambda: None)
    ok = True
    for dtype in (torch.float32, torch.bfloat16):
        c = SymmCollective(1 << 20, dtype, dev)
        g = torch.Generator(device="cpu").manual_seed(7 + rank)
        x = torch.randn(c.numel, generator=g).to(dtype).to(dev)
        for average in (False, True):
            c.tensor.copy_(x)
            ref = x.float().clone()
            dist.all_reduce(ref)
            if average:
                ref /= world
            c.all_reduce_(average=average)
            sync()
            tol = 1e-5 if dtype == torch.float32 else 3e-2
            err = (c.tensor.float() - ref).abs().max().item()
            ok = ok and err <= tol * max(1.0, ref.abs().max().item())
        # the result is the same bits on every rank
        chk = c.tensor.float().clone()
        dist.broadcast(chk, src=0)
        ok = ok and torch.equal(chk, c.tensor.float())
        # sub-range, captured in a graph and replayed with new data
        per = 16 * world // c.esize
        off, n = 3 * per, 1000 * per
        c.tensor.copy_(x)
        c.all_reduce_(numel=n, offset=off)                     # warm-up outside of the capture
        sync()
        if on_gpu:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                c.all_reduce_(numel=n, offset=off)
            replay = graph.replay
        else:
            replay = lambda: c.all_reduce_(numel=n, offset=off)
        for it in range(2):
            y = (x * (it + 2)).to(dtype)
            c.tensor.copy_(y)
            replay()
            sync()
            ref = y.float()[off:off + n].clone()
            dist.all_reduce(ref)
            tol = 1e-5 if dtype == torch.float32 else 3e-2
            ok = ok and (c.tensor.float()[off:off + n] - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
            ok = ok and torch.equal(c.tensor[:off], y[:off]) and torch.equal(c.tensor[off + n:], y[off + n:])
        # all-gather
        c.tensor.zero_()
        sl = c.numel // world
        c.tensor[rank * sl:(rank + 1) * sl] = x[rank * sl:(rank + 1) * sl]
        c.all_gather_()
        sync()
        parts = [torch.empty(sl, dtype=dtype, device=dev) for _ in range(world)]
        dist.all_gather(parts, x[rank * sl:(rank + 1) * sl].contiguous())
        ok = ok and torch.equal(c.tensor, torch.cat(parts))
        print(f"rank {rank}: {dtype} multimem={'yes' if (c.buf is not None and c.buf.mc_ptr) else 'no'} ok={ok}", flush=True)

    # plain data parallelism: symmetric all-reduce against NCCL
    finals = []
    for comm in ("nccl", "symm"):
        torch.manual_seed(3)
        net = torch.nn.Sequential(torch.nn.Linear(256, 512), torch.nn.GELU(), torch.nn.Linear(512, 64)).to(dev).to(torch.bfloat16)
        opt = AllReduceOptimizer(net.parameters(), lr=1e-2, weight_decay=0.1, comm=comm)
        for step in range(4):
            xb = torch.randn(32, 256, generator=torch.Generator().manual_seed(100 * step + rank)).to(dev).to(torch.bfloat16)
            opt.zero_grad()
            for p in opt.params:
                p.grad = None
            net(xb).float().pow(2).mean().backward()
            opt.step()
        sync()
        finals.append(torch.cat([p.detach().float().flatten() for p in net.parameters()]))
    e = (finals[0] - finals[1]).abs().max().item()
    ok = ok and e < 2e-2
    # weights sharded by rows, gathered inside the forward GEMM, updated by the owner only
    from tinyinfinitrain_b200.parallel.param_gather import GatheredWeightLinear, RowShardedAdam

    D, H = 256, 128 * world
    l1 = GatheredWeightLinear(D, H, device=dev)
    l2 = GatheredWeightLinear(H, 128 * world, device=dev)
    l2.reset_parameters(seed=7)
    g1 = torch.Generator().manual_seed(42)
    ref1, ref2 = torch.nn.Linear(D, H), torch.nn.Linear(H, 128 * world)
    with torch.no_grad():       # the layers draw (weight, bias) from a seeded generator: rebuild the same values
        b1 = 1.0 / D ** 0.5
        ref1.weight.copy_((torch.rand(H, D, generator=g1) * 2 - 1) * b1); ref1.bias.copy_((torch.rand(H, generator=g1) * 2 - 1) * b1)
        g2, b2 = torch.Generator().manual_seed(7), 1.0 / H ** 0.5
        ref2.weight.copy_((torch.rand(128 * world, H, generator=g2) * 2 - 1) * b2)
        ref2.bias.copy_((torch.rand(128 * world, generator=g2) * 2 - 1) * b2)
    ref1, ref2 = ref1.to(dev), ref2.to(dev)
    w_init = l1.weight[l1.own_rows()].float().clone()
    popt = RowShardedAdam([l1, l2], lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    ropt = torch.optim.AdamW(list(ref1.parameters()) + list(ref2.parameters()), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    for step in range(3):
        xs = [torch.randn(64, D, generator=torch.Generator().manual_seed(10 * step + r)).to(dev) for r in range(world)]
        popt.zero_grad()
        y = l2(torch.tanh(l1(xs[rank].to(torch.bfloat16))))
        ok = ok and bool(torch.isfinite(y.float()).all())          # unfetched rows would be NaN
        y.float().pow(2).mean().backward()
        popt.step()
        ropt.zero_grad()
        (sum(ref2(torch.tanh(ref1(x))).pow(2).mean() for x in xs) / world).backward()
        ropt.step()
    sync()
    ew = max((l.weight[l.own_rows()].float() - r.weight[l.own_rows()].detach()).abs().max().item() for l, r in ((l1, ref1), (l2, ref2)))
    moved = (l1.weight[l1.own_rows()].float() - w_init).abs().max().item()
    ok = ok and ew < 8e-3 and moved > 1e-3        # near-zero gradients may flip sign in bf16: up to 2 lr per step apart
    print(f"rank {rank}: row-sharded layers vs replicated fp32 AdamW max|dw|={ew:.3e} ok={ok}", flush=True)
    status = C.status_read(True) if on_gpu else 0
    ok = ok and status == 0
    print(f"rank {rank}: data-parallel nccl-vs-symm max|dp|={e:.3e} status={status} ok={ok}", flush=True)
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if t.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
