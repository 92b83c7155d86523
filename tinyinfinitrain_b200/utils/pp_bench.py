"""Bubble fraction of the 1F1B pipeline schedule, measured (run under torchrun, one rank per GPU, world = stages).

    torchrun --nproc-per-node 2 -m tinyinfinitrain_b200.utils.pp_bench --micro 8

The schedule is timed with m and with 2m micro-batches (forward + backward of every micro-batch, no optimizer;
CUDA events, maximum over ranks).  With P stages an ideal 1F1B step lasts (m + P - 1) slots, one slot being the
forward + backward of one micro-batch on the slowest stage, so

    slot      = (T(2m) - T(m)) / m
    bubble(m) = (T(m) - m * slot) / T(m)          ideal: (P - 1) / (m + P - 1)

A bubble above the ideal value means time lost to exposed sends / receives or to stages of unequal cost; rank 0
prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main():
    from ..models import GPT2Config
    from .train import ParallelTrainStep

    ap = argparse.ArgumentParser()
    ap.add_argument("--micro", type=int, default=8, help="m: micro-batches of the shorter run")
    ap.add_argument("--batch", type=int, default=4, help="sequences per micro-batch")
    ap.add_argument("--seq", type=int, default=1024)
    ap.add_argument("--layers", type=int, default=12)
    ap.add_argument("--d_model", type=int, default=768)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--json_out", default="")
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("LOCAL_RANK", 0))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("nccl", device_id=dev)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("gloo")
    cfg = GPT2Config(block_size=a.seq, n_layer=a.layers, n_head=a.heads, n_embd=a.d_model)
    m = a.micro
    step = ParallelTrainStep(cfg, a.batch, a.seq, dev, dtype=torch.bfloat16 if cuda else torch.float32, tp=1, pp=world,
                             num_microbatches=2 * m, zero_stage=0)
    g = torch.Generator().manual_seed(1)
    for x, y in step.batches:
        x.copy_(torch.randint(0, cfg.vocab_size, x.shape, generator=g))
        y.copy_(torch.randint(0, cfg.vocab_size, y.shape, generator=g))

    def timed(n_micro: int) -> float:
        import time

        for _ in range(2):
            step.opt.zero_grad()
            step.stage.run(n_micro)
        if cuda:
            torch.cuda.synchronize()
        dist.barrier()
        if cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        t0 = time.perf_counter()
        for _ in range(a.iters):
            step.opt.zero_grad()
            step.stage.run(n_micro)
        if cuda:
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / a.iters
        else:
            ms = (time.perf_counter() - t0) * 1e3 / a.iters
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    t1, t2 = timed(m), timed(2 * m)
    slot = (t2 - t1) / m
    rec = {"stages": world, "micro_batches": m, "tokens_per_micro_batch": a.batch * a.seq,
           "model": f"gpt2 L{a.layers} d{a.d_model}", "ms_m": t1, "ms_2m": t2, "slot_ms": slot,
           "bubble_measured": (t1 - m * slot) / t1, "bubble_ideal": (world - 1) / (m + world - 1),
           "bubble_measured_2m": (t2 - 2 * m * slot) / t2, "bubble_ideal_2m": (world - 1) / (2 * m + world - 1)}
    if rank == 0:
        print(json.dumps(rec), flush=True)
        if a.json_out:
            with open(a.json_out, "w") as f:
                json.dump(rec, f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
