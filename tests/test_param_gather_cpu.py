"""Row-sharded weights gathered by the consuming layer + RowShardedAdam, over two and three gloo ranks: the training
trajectory equals a single replicated model trained with AdamW on the ranks' averaged gradients."""
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
        from tinyinfinitrain_b200.parallel.param_gather import GatheredWeightLinear, RowShardedAdam

        D, H = 10, 6 * world
        l1 = GatheredWeightLinear(D, H, dtype=torch.float32)
        l2 = GatheredWeightLinear(H, 3 * world, dtype=torch.float32)
        l2.reset_parameters(seed=7)
        ref1, ref2 = torch.nn.Linear(D, H), torch.nn.Linear(H, 3 * world)
        with torch.no_grad():
            ref1.weight.copy_(l1.weight); ref1.bias.copy_(l1.bias)
            ref2.weight.copy_(l2.weight); ref2.bias.copy_(l2.bias)
        # a rank's copy of the rows it does not own is stale until the layer gathers them
        with torch.no_grad():
            for l in (l1, l2):
                keep = l.weight[l.own_rows()].clone()
                l.weight.fill_(123.0)
                l.weight[l.own_rows()] = keep
        opt = RowShardedAdam([l1, l2], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
        ropt = torch.optim.AdamW(list(ref1.parameters()) + list(ref2.parameters()), lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
        ok = True
        for step in range(4):
            xs = [torch.randn(5, D, generator=torch.Generator().manual_seed(10 * step + r)) for r in range(world)]
            opt.zero_grad()
            y = l2(torch.tanh(l1(xs[rank])))
            y.pow(2).mean().backward()
            opt.step()
            ropt.zero_grad()
            loss = sum(ref2(torch.tanh(ref1(x))).pow(2).mean() for x in xs) / world
            loss.backward()
            ropt.step()
            for l, r in ((l1, ref1), (l2, ref2)):
                ok &= torch.allclose(l.weight[l.own_rows()], r.weight[l.own_rows()].detach(), atol=1e-5)
                ok &= torch.allclose(l.bias, r.bias.detach(), atol=1e-5)
        # one more forward refreshes every rank's full copy
        l2(torch.tanh(l1(xs[rank])))
        ok &= torch.allclose(l1.weight, ref1.weight.detach(), atol=1e-5) and torch.allclose(l2.weight, ref2.weight.detach(), atol=1e-5)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_sharded_training_matches_replicated_adamw(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 200 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=240) for _ in range(world)]
    for p in procs:
        p.join(60)
    assert all(ok for _, ok in res), res


def test_tile_order_of_the_gather_kernel_covers_every_tile_once():
    """Emulates tile_coord for collective mode 3: n-blocks rotated so that the local shard comes first."""
    for world in (1, 2, 4, 8):
        for rows_per_rank, bn in ((128, 128), (256, 256), (384, 128), (512, 256)):
            N = rows_per_rank * world
            tiles_n, tiles_m = (N + bn - 1) // bn, 5
            for rank in range(world):
                seen, first_n = set(), None
                for mn in range(tiles_m * tiles_n):
                    mblk = mn % tiles_m
                    nblk = (mn // tiles_m + (rank * rows_per_rank) // bn) % tiles_n
                    if first_n is None:
                        first_n = nblk
                    seen.add((mblk, nblk))
                assert len(seen) == tiles_m * tiles_n
                assert first_n * bn == rank * rows_per_rank            # starts on the rows this rank owns
