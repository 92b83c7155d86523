"""Worker for the multi-GPU ZeRO-1 test: launched by torchrun, one rank per GPU.

Trains a small GPT-2 for a few steps with the fused NVLink step (reduce-scatter + Adam +
all-gather in one kernel) and with the NCCL baseline, from identical initial weights and data,
and checks that the two parameter sets agree and that the loss falls.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def run(comm, steps, dev, rank, use_graph=False, buckets=1, clip=0.0):
    import tinyinfinitrain_b200 as tit
    from tinyinfinitrain_b200.models import GPT2, GPT2Config
    from tinyinfinitrain_b200.utils import TrainStep

    cfg = GPT2Config(block_size=128, vocab_size=1000, n_layer=2, n_head=4, n_embd=256)
    model = GPT2(cfg, device=dev, dtype=torch.bfloat16, seed=42)
    opt = tit.parallel.DistributedOptimizer(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1, comm=comm,
                                            num_buckets=buckets, overlap=buckets > 1, max_grad_norm=clip)
    step = TrainStep(model, opt, 4, 128, dev, use_graph=use_graph)
    g = torch.Generator().manual_seed(1234 + rank)
    idx = torch.randint(0, 1000, (4, 128), generator=g).pin_memory()
    tgt = torch.roll(idx, -1, 1).pin_memory()
    losses = []
    if use_graph:
        step.idx.copy_(idx); step.tgt.copy_(tgt)
        step.prepare(eager_warmup=1)
    for _ in range(steps):
        hl = step(idx, tgt)
        torch.cuda.synchronize()
        losses.append(float(hl))
    status = tit._lib.C.status_read(True)
    return opt.flat.param.float().clone(), losses, status, opt


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    p_nccl, l_nccl, s0, _ = run("nccl", 6, dev, rank)
    p_fused, l_fused, s1, opt = run("fused", 6, dev, rank)
    p_graph, l_graph, s2, _ = run("fused", 5, dev, rank, use_graph=True)  # 1 eager warm-up + 5 replays = 6 steps
    err = (p_nccl - p_fused).abs().max().item()
    errg = (p_fused - p_graph).abs().max().item()
    # every rank must hold identical parameters after the all-gather
    ref = p_fused.clone()
    dist.broadcast(ref, src=0)
    same = bool((ref - p_fused).abs().max().item() == 0.0)
    ok = s0 == 0 and s1 == 0 and s2 == 0 and err < 2e-2 and errg < 2e-2 and same and l_fused[-1] < l_fused[0] - 0.3
    nb = int(os.environ.get("TITB_TEST_ZERO_BUCKETS", "0"))
    if nb > 1:
        # bucketed reduction launched from backward on a side stream: same arithmetic, so the same parameters
        p_b, l_b, s3, ob = run("fused", 6, dev, rank, buckets=nb)
        p_bg, l_bg, s4, _ = run("fused", 5, dev, rank, use_graph=True, buckets=nb)
        eb, ebg = (p_fused - p_b).abs().max().item(), (p_fused - p_bg).abs().max().item()
        early = sum(1 for b in ob.buckets if not b["late"])
        ok = ok and s3 == 0 and s4 == 0 and eb < 2e-2 and ebg < 2e-2 and len(ob.buckets) > 1 and early >= 1
        print(f"rank {rank}: buckets={len(ob.buckets)} reduced-during-backward={early} fused-vs-bucketed={eb:.3e} "
              f"bucketed-graph={ebg:.3e} status={s3},{s4}", flush=True)
    clip = float(os.environ.get("TITB_TEST_ZERO_CLIP", "0"))
    if clip > 0:
        # global-norm clipping: fused (NVLink norm pass + local scaling) against the unfused NCCL path, eager and captured
        p_cn, _, s5, on = run("nccl", 6, dev, rank, clip=clip)
        p_cf, _, s6, of = run("fused", 6, dev, rank, clip=clip)
        p_cg, _, s7, _ = run("fused", 5, dev, rank, use_graph=True, clip=clip)
        ec, ecg = (p_cn - p_cf).abs().max().item(), (p_cf - p_cg).abs().max().item()
        nn_, nf = on.grad_norm(), of.grad_norm()
        moved = (p_cf - p_fused).abs().max().item()          # clipping changed the trajectory
        ok = ok and s5 == 0 and s6 == 0 and s7 == 0 and ec < 2e-2 and ecg < 2e-2 and abs(nn_ - nf) < 2e-2 * max(1.0, nn_) \
            and moved > 0
        print(f"rank {rank}: clip nccl-vs-fused={ec:.3e} fused-vs-graph={ecg:.3e} norms {nn_:.4f} / {nf:.4f}", flush=True)
    print(f"rank {rank}: nccl-vs-fused max|dp|={err:.3e} fused-vs-graph={errg:.3e} identical_across_ranks={same} "
          f"status={s0},{s1},{s2} multimem={'yes' if opt.gbuf.mc_ptr else 'no'} loss {l_fused[0]:.3f}->{l_fused[-1]:.3f} "
          f"ok={ok}", flush=True)
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if t.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
