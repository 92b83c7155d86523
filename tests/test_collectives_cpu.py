"""Standalone symmetric-memory collectives: host-side logic (padding, range checks, the gloo fallback that shares
the call signature with the CUDA kernels) over two and three CPU ranks, and a PyTorch emulation of the slice
arithmetic of csrc/kernels/collectives.cu (which rank reduces / writes which bytes)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from tinyinfinitrain_b200.parallel.collectives import SymmCollective, padded_numel

        ok = True
        c = SymmCollective(1000, torch.float32, "cpu")
        ok &= c.numel == padded_numel(1000, torch.float32, world) and c.numel % (4 * world) == 0 and c.numel >= 1000
        c.tensor.copy_(torch.arange(c.numel, dtype=torch.float32) * (rank + 1))
        c.all_reduce_(average=True)
        want = torch.arange(c.numel, dtype=torch.float32) * sum(r + 1 for r in range(world)) / world
        ok &= torch.allclose(c.tensor, want)
        # all-gather of a sub-range: every rank fills its own slice only
        n = 8 * world
        c.tensor.zero_()
        per = n // world
        c.tensor[16 + rank * per:16 + (rank + 1) * per] = float(rank + 1)
        c.all_gather_(numel=n, offset=16)
        want = torch.cat([torch.full((per,), float(r + 1)) for r in range(world)])
        ok &= torch.equal(c.tensor[16:16 + n], want) and float(c.tensor[:16].abs().sum()) == 0.0
        try:
            c.all_reduce_(numel=4 * world, offset=3)        # misaligned offset
            ok = False
        except ValueError:
            pass
        # plain data parallelism: asking for the symmetric path on CPU parameters falls back to the process group
        from tinyinfinitrain_b200.parallel import AllReduceOptimizer

        torch.manual_seed(0)
        lin = torch.nn.Linear(9, 5)
        opt = AllReduceOptimizer(lin.parameters(), lr=1e-2, comm="symm")
        ok &= opt.coll is None
        lin(torch.randn(3, 9, generator=torch.Generator().manual_seed(rank))).sum().backward()
        opt.step()
        w = lin.weight.detach().clone()
        dist.all_reduce(w)
        ok &= torch.allclose(w / world, lin.weight.detach(), atol=1e-6)      # replicas stayed identical
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_symm_collective_cpu_fallback(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29300 + os.getpid() % 200 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(60)
    assert all(ok for _, ok in res), res


def test_slice_arithmetic_of_the_kernels():
    """Each rank handles slice_vecs = nbytes / 16 / world vectors starting at byte_off / 16 + rank * slice_vecs:
    the slices tile the range exactly once, so the in-place all-reduce never reads what another rank writes."""
    for world in (1, 2, 3, 4, 8, 16):
        for vec_per_rank in (1, 5, 1000):
            nbytes, byte_off = 16 * world * vec_per_rank, 48
            covered = torch.zeros(byte_off // 16 + nbytes // 16 + 2, dtype=torch.int32)
            for rank in range(world):
                sv = nbytes // 16 // world
                so = byte_off // 16 + sv * rank
                covered[so:so + sv] += 1
            assert int(covered[:byte_off // 16].sum()) == 0 and int(covered[-2:].sum()) == 0
            assert torch.all(covered[byte_off // 16:byte_off // 16 + nbytes // 16] == 1)


def test_multi_gpu_check_script_dry_run_over_gloo():
    """tests/dist_collectives_check.py, the job the multi-GPU test launches, with TITB_TEST_DEVICE=cpu: the script's own
    logic (references, tolerances, call signatures) runs over two gloo ranks and the CPU fallbacks of the same classes."""
    from _launch import run_group

    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(29150 + os.getpid() % 40), os.path.join(ROOT, "tests", "dist_collectives_check.py")]
    r = run_group(cmd, env=dict(os.environ, TITB_TEST_DEVICE="cpu"), timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "row-sharded layers" in r.stdout and "ok=True" in r.stdout
