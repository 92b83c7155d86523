#!/usr/bin/env python
"""Training-throughput benchmark (tokens/s), bf16 compute + fp32 master weights, synthetic uniform token ids.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W [--config NAME]

``--config`` (default ``gpt2_dp``):

    gpt2_dp             GPT-2 124M, micro-batch 8 x 1024 per GPU, AdamW, data parallel + ZeRO-1 over the N GPUs
    llama1b_tp8         LLaMA-3-style 1B, batch 4 x 2048, tensor + sequence parallel over all N GPUs
    gpt2xl_tp2pp2dp2    GPT-2 XL 1.5B, T 1024, TP2 x PP2 x DP(N/4), 1F1B with 8 micro-batches of 4
    llama8b_tp4dp2      LLaMA-3 8B, T 4096, global batch 16, TP4 x DP(N/4) + ZeRO-1, 8 micro-batches of 1 per replica

Rank 0 prints one JSON line.  ``value`` is device-timed (CUDA events, max over ranks) with the batch already
resident; ``e2e`` times the public step call (``TrainStep.__call__`` / ``ParallelTrainStep.__call__``) including the
pinned host->device copy of every step's tokens and the device->host read of every step's loss.  The default arm
also runs the comparison arm of its config in the same process group right after its own measurement -- for
``gpt2_dp`` the library arm (stock PyTorch: cuBLAS, SDPA, fused AdamW, DDP over NCCL; none of this repository's
kernels), for the tensor-parallel configs this repository's kernels with plain NCCL collectives instead of the
fused ones -- and reports ``vs_baseline`` = own value / that arm's value (``--no-baseline`` skips it).
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CONFIGS = {
    # name: family, preset, micro-batch, seq, tp (0 = all GPUs), pp, micro-batches per step, zero stage
    "gpt2_dp": dict(family="gpt2", preset="gpt2", label="gpt2-124M", B=8, T=1024, tp=1, pp=1, nm=1),
    "llama1b_tp8": dict(family="llama3", preset="llama3-1b", label="llama3-1B", B=4, T=2048, tp=0, pp=1, nm=1),
    "gpt2xl_tp2pp2dp2": dict(family="gpt2", preset="gpt2-xl", label="gpt2-xl-1.5B", B=4, T=1024, tp=2, pp=2, nm=8),
    "llama8b_tp4dp2": dict(family="llama3", preset="llama3-8b", label="llama3-8B", B=1, T=4096, tp=4, pp=1, nm=8),
}


def reference_arm(args):
    # The reference tree has no setup.py/pyproject.toml, its four submodules (glog, gflags, eigen,
    # googletest) are empty directories, and 13 of its functions are unimplemented stubs, so it can
    # neither be installed nor built offline.
    if int(os.environ.get("RANK", "0")) != 0:  # under torchrun only rank 0 reports
        return 0
    print(json.dumps({"impl": "reference",
                      "unavailable": "reference is not installable (no setup.py/pyproject.toml; pip: 'Neither setup.py "
                                     "nor pyproject.toml found'), its third_party submodules are empty and its kernel "
                                     "registry, Matmul, Adam and Tensor::Backward are unimplemented stubs"}))
    return 0


class WallEvent:  # stands in for a CUDA event on the CPU dry run
    def record(self):
        self.t = time.perf_counter()

    def elapsed_time(self, other):
        return (other.t - self.t) * 1e3


def measure(ctx, make_step, K, W, sample_clocks):
    """Builds a step object with ``make_step()`` and times it twice: K device-timed steps on resident inputs, then K
    end-to-end steps through its ``__call__``.  Returns a dict of raw results (times are max over ranks)."""
    import torch

    dev, world, on_gpu = ctx["dev"], ctx["world"], ctx["on_gpu"]
    step, host_batches = make_step()

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        if on_gpu:
            torch.cuda.synchronize(dev)

    def new_event():
        return torch.cuda.Event(enable_timing=True) if on_gpu else WallEvent()

    sampler = None
    if sample_clocks and ctx["rank"] == 0:
        from tinyinfinitrain_b200.utils.clocks import ClockSampler

        uuid = str(getattr(torch.cuda.get_device_properties(dev), "uuid", "") or "") if on_gpu else ""
        sampler = ClockSampler(ctx["local_rank"], uuid=uuid)
        sampler.launch()

    # ---------------- device-timed region: K steps, inputs resident -----------------
    for _ in range(W):
        step.run_device()
    barrier()
    if sampler is not None:
        sampler.begin()
    e0, e1 = new_event(), new_event()
    e0.record()
    for _ in range(K):
        step.run_device()
    e1.record()
    barrier()
    if sampler is not None:
        sampler.end()
    ms = e0.elapsed_time(e1)
    final_loss = float(step.loss)

    # ---------------- end-to-end region: H2D of tokens + step + D2H of loss, every step -----------------
    nbuf = len(host_batches)
    for i in range(3):
        step(*host_batches[i % nbuf])
    barrier()
    t0 = time.perf_counter()
    for i in range(K):
        hl = step(*host_batches[i % nbuf])
        if on_gpu:
            torch.cuda.current_stream().synchronize()
        _ = float(hl)
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1e3

    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = t.tolist()
        # the loss lives on the last pipeline stage: take the largest value any rank reports (others hold 0)
        lt = torch.tensor([final_loss], device=dev, dtype=torch.float64)
        dist.all_reduce(lt, op=dist.ReduceOp.MAX)
        final_loss = float(lt)
    out = {"ms": ms, "e2e_ms": e2e_ms, "final_loss": final_loss, "step": step,
           "clocks": sampler.result() if sampler is not None else None}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "library"],
                    help="ours: this framework; reference: the unmodified reference (unavailable, see above); "
                         "library: stock PyTorch modules (cuBLAS, SDPA, fused AdamW, DDP/NCCL) on the gpt2_dp config")
    ap.add_argument("--config", default="gpt2_dp", choices=sorted(CONFIGS))
    ap.add_argument("--model", default="", help="override the preset name of the config's model family")
    ap.add_argument("--batch", type=int, default=0, help="override the micro-batch per GPU / per replica")
    ap.add_argument("--seq", type=int, default=0)
    ap.add_argument("--tp", type=int, default=-1, help="override the tensor-parallel degree of the config (dry runs on fewer GPUs)")
    ap.add_argument("--pp", type=int, default=-1)
    ap.add_argument("--micro", type=int, default=0, help="override the micro-batches per step")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (reported; not the named config any more)")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-baseline", action="store_true", help="skip the comparison arm (vs_baseline stays null)")
    ap.add_argument("--dp_buckets", type=int, default=1,
                    help="ZeRO-1 buckets; >1 reduces each bucket on a side stream as soon as backward has written it")
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"],
                    help="cpu = dry run of this script's control flow (gloo ranks, fp32, wall-clock timing); not a benchmark")
    ap.add_argument("--tiny", action="store_true", help="2-layer 64-wide model for dry runs (reported as such)")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="collectives of the own arm: this repository's NVLink kernels, or plain NCCL")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    import dataclasses

    import torch

    import tinyinfinitrain_b200 as tit
    from tinyinfinitrain_b200.models import GPT2, GPT2_PRESETS, LLAMA3_PRESETS
    from tinyinfinitrain_b200.utils import ParallelTrainStep, TrainStep

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus or world == 1 and args.gpus == 1, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    on_gpu = args.device == "cuda"
    if on_gpu:
        torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank) if on_gpu else torch.device("cpu")
    dtype = torch.bfloat16 if on_gpu else torch.float32
    W = max(3, args.warmup)
    K = args.steps
    ctx = {"dev": dev, "world": world, "rank": rank, "local_rank": local_rank, "on_gpu": on_gpu}

    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if on_gpu:
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")

    spec = dict(CONFIGS[args.config])
    presets = GPT2_PRESETS if spec["family"] == "gpt2" else LLAMA3_PRESETS
    cfg = dataclasses.replace(presets[args.model or spec["preset"]])
    label = spec["label"] if not args.model else args.model
    if args.tiny:
        from tinyinfinitrain_b200.models import GPT2Config, LLaMA3Config

        cfg = GPT2Config(block_size=max(32, args.seq), vocab_size=1000, n_layer=2, n_head=4, n_embd=64) \
            if spec["family"] == "gpt2" else \
            LLaMA3Config(block_size=max(32, args.seq), vocab_size=1024, n_layer=2, n_head=16, n_kv_head=8, n_embd=128, ffn_dim=256)
        label = f"{spec['family']}-tiny (dry run)"
    if args.layers:
        cfg.n_layer = args.layers
        label += f" cut to {args.layers} layers (not the named config)"
    B, T = args.batch or spec["B"], args.seq or spec["T"]
    cfg.block_size = max(cfg.block_size, T)
    tp = spec["tp"] if args.tp < 0 else args.tp
    tp = world if tp == 0 else tp
    pp = spec["pp"] if args.pp < 0 else args.pp
    nm = args.micro or spec["nm"]
    parallel_path = (args.config != "gpt2_dp") or tp > 1 or pp > 1
    assert world % (tp * pp) == 0, f"{world} GPUs do not divide into tp{tp} x pp{pp}"
    dp = world // (tp * pp)
    library = args.impl == "library"
    if library and parallel_path:
        raise SystemExit("--impl library exists for the gpt2_dp config only; the comparison arm of the other configs is --comm nccl")

    # synthetic uniform token ids, pinned on the host: seed 0 + data-parallel rank, so that replicas see different data
    # and the tensor / pipeline ranks of one replica see the same batch
    nbuf = 4
    gen = torch.Generator().manual_seed(0 + rank // (tp * pp))
    pin = (lambda t: t.pin_memory()) if on_gpu else (lambda t: t)

    def host_pair():
        x = torch.randint(0, cfg.vocab_size, (B, T), generator=gen)
        return pin(x), pin(torch.roll(x, -1, dims=1))

    if not parallel_path:
        host = [host_pair() for _ in range(nbuf)]
    else:
        host = [([host_pair() for _ in range(nm)],) for _ in range(nbuf)]

    def make_ours(comm):
        def make():
            if not parallel_path:
                model = GPT2(cfg, device=dev, dtype=dtype, seed=42)
                if world == 1:
                    opt = tit.optim.MixedPrecisionAdam(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
                else:
                    from tinyinfinitrain_b200 import parallel

                    # the distributed optimizer's step() owns reduce-scatter / Adam / all-gather
                    opt = parallel.DistributedOptimizer(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1,
                                                        comm=comm, num_buckets=args.dp_buckets, overlap=args.dp_buckets > 1)
                # the NCCL arm runs eagerly: its collectives are library calls issued per step, not captured
                use_graph = not args.no_graph and (world == 1 or comm == "fused")
                step = TrainStep(model, opt, B, T, dev, use_graph=use_graph)
                step.idx.copy_(host[0][0]); step.tgt.copy_(host[0][1])
                step.prepare()
                return step, host
            step = ParallelTrainStep(cfg, B, T, dev, dtype, tp=tp, pp=pp, num_microbatches=nm, zero_stage=1, comm=comm,
                                     dp_buckets=args.dp_buckets, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1, seed=42,
                                     exact_init_limit=0 if on_gpu else 1 << 26)
            for (x, y), (hx, hy) in zip(step.batches, host[0][0]):
                x.copy_(hx); y.copy_(hy)
            return step, host
        return make

    def make_library():
        from baseline.library_gpt2 import LibraryGPT2, LibraryTrainStep

        model = LibraryGPT2(cfg.vocab_size, cfg.padded_vocab_size, cfg.block_size, cfg.n_layer, cfg.n_head, cfg.n_embd)
        # same starting point as the hand-written arm: its seeded initialisation, copied by name
        model.load_named(GPT2(cfg, device="cpu", dtype=torch.float32, seed=42).StateDict())
        model = model.to(dev)
        step = LibraryTrainStep(model, B, T, dev, world)
        step.idx.copy_(host[0][0]); step.tgt.copy_(host[0][1])
        return step, host

    tokens_per_step = B * T * nm * dp if parallel_path else B * T * world
    res = measure(ctx, make_library if library else make_ours(args.comm), K, W, sample_clocks=True)
    step = res["step"]
    status = tit._lib.C.status_read(True) if (on_gpu and not library) else 0
    launches = 0 if library else int(step.launches_per_step) * K
    opt = getattr(step, "opt", None)
    nvls = bool(getattr(getattr(opt, "gbuf", None), "mc_ptr", 0)) if not library else False
    graph = getattr(step, "graph", None) is not None

    # ---------------- comparison arm of this config, same process group, same steps -----------------
    base = None
    if args.impl == "ours" and not args.no_baseline and not (parallel_path and args.comm == "nccl"):
        del step, opt
        res["step"] = None
        gc.collect()
        if on_gpu:
            torch.cuda.empty_cache()
        b = measure(ctx, make_ours("nccl") if parallel_path else make_library, K, W, sample_clocks=True)
        b.pop("step")
        gc.collect()
        base = {"impl": "own kernels + NCCL collectives (--comm nccl)" if parallel_path
                else "library (cuBLAS, SDPA, fused AdamW, DDP/NCCL; bench.py --impl library)",
                "value": tokens_per_step * K / (b["ms"] / 1e3), "ms_per_step": b["ms"] / K,
                "e2e_value": tokens_per_step * K / (b["e2e_ms"] / 1e3), "final_loss": b["final_loss"], "clocks": b["clocks"]}

    if rank == 0:
        clocks = res["clocks"]
        ms, e2e_ms = res["ms"], res["e2e_ms"]
        value = tokens_per_step * K / (ms / 1e3)
        e2e_value = tokens_per_step * K / (e2e_ms / 1e3)
        if parallel_path:
            par = "+".join(x for x in (f"tp{tp}" + ("+sp" if tp > 1 else ""), f"pp{pp}" if pp > 1 else "", f"dp{dp}" + ("+zero1" if dp > 1 else "")) if x)
        else:
            par = f"dp{world}" + ("+zero1" if world > 1 and not library else "")
        out = {
            "metric": "train_tokens_per_sec", "value": value, "unit": "tokens/s",
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms / K, "higher_is_better": True,
            "scaling": "weak" if not parallel_path else "strong",
            "vs_baseline": (value / base["value"]) if base else None,
            "dtype": "bf16" if on_gpu else "fp32 (cpu dry run)", "data": "synthetic",
            "config": {"name": args.config, "model": label, "global_batch": tokens_per_step // T, "seq_len": T,
                       "parallelism": par, "micro_batch_per_gpu": B, "micro_batches_per_step": nm,
                       "optimizer": "AdamW(fp32 params, bf16 autocast)" if library else "AdamW(fp32 master, bf16 params)",
                       "cuda_graph": graph,
                       "comm": ("nccl-ddp" if library else args.comm) if world > 1 else "none",
                       "nvls_multimem": nvls,
                       "l2": "per-step working set (activations + weights + optimizer state, >10 GB) exceeds the "
                             "126 MB L2; no explicit flush",
                       "init": "random N(0,0.02), seed 42", "final_loss": res["final_loss"], "kernel_status": status,
                       # kernel variants switched on through the environment for this run (empty = defaults)
                       "switches": {k: v for k, v in sorted(os.environ.items()) if k.startswith("TITB200_")}},
            "clocks": {"sm_mhz": clocks["sm_mhz"], "sm_max_mhz": clocks["sm_max_mhz"], "reasons": clocks["reasons"],
                       "samples": clocks["samples"], "source": clocks["backend"]},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 2 * B * T * 8 * (nm if parallel_path else 1),
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / K,
                    "vs_baseline": (e2e_value / base["e2e_value"]) if base else None},
            # launches of this repository's own kernels inside the timed region (none on the library arm)
            "gpu_launches": launches,
            "impl": args.impl,
        }
        if base:
            bc = base.pop("clocks")
            base["clocks"] = {"sm_mhz": bc["sm_mhz"], "sm_max_mhz": bc["sm_max_mhz"], "reasons": bc["reasons"], "samples": bc["samples"]}
            # loss of both arms after the same number of steps from the same weights on the same batches
            base["loss_gap"] = abs(base["final_loss"] - res["final_loss"])
            out["baseline"] = base
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
