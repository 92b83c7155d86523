"""Training entry point shared by ``examples/gpt2/main.py`` and ``examples/llama3/main.py``.

Flag names follow the fixture fields of the reference's end-to-end test
(test/example/test_gpt2.cc:106-119) and the flag names its sources hint at
(``FLAGS_batch_size, FLAGS_sequence_length``, example/common/tokenizer.cc:95), extended with the
parallelism and precision switches of this framework.  Run under ``torchrun`` for more than one
GPU; ranks are laid out as dp x pp x tp (``parallel/mesh.py``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def build_parser(family: str) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description=f"Train {family} with tinyinfinitrain_b200")
    p.add_argument("--llmc_filepath", default="", help="llm.c checkpoint to start from (random init if empty)")
    p.add_argument("--input_bin", default="", help="llm.c token file (.bin); synthetic tokens if empty")
    p.add_argument("--tokenizer_bin", default="", help="llm.c tokenizer file, enables text generation")
    p.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    p.add_argument("--model", default="gpt2" if family == "gpt2" else "llama3-1b")
    p.add_argument("--batch_size", type=int, default=4, help="micro-batch per data-parallel rank")
    p.add_argument("--sequence_length", type=int, default=64)
    p.add_argument("--total_batch_size", type=int, default=0, help="tokens per optimizer step (0 = one micro-batch)")
    p.add_argument("--num_iteration", type=int, default=10)
    p.add_argument("--text_length", type=int, default=64)
    p.add_argument("--freq_generate_txt", type=int, default=0)
    p.add_argument("--learning_rate", type=float, default=1e-4)
    p.add_argument("--weight_decay", type=float, default=0.0)
    p.add_argument("--max_grad_norm", type=float, default=0.0, help="clip the global gradient norm (0 = off)")
    p.add_argument("--warmup_steps", type=int, default=0, help="linear learning-rate warm-up steps")
    p.add_argument("--lr_decay_steps", type=int, default=0, help="cosine decay horizon in steps (0 = constant rate)")
    p.add_argument("--min_lr_ratio", type=float, default=0.1, help="final rate of the cosine decay / peak rate")
    p.add_argument("--optimizer", default="adam", choices=["adam", "sgd"])
    p.add_argument("--dtype", default="bfloat16", choices=["float32", "bfloat16"])
    p.add_argument("--tensor_parallel", type=int, default=1)
    p.add_argument("--sequence_parallel", type=int, default=1, help="kept for flag parity: TP always runs sequence parallel")
    p.add_argument("--pipeline_parallel", type=int, default=1)
    p.add_argument("--num_microbatches", type=int, default=1)
    p.add_argument("--zero_stage", type=int, default=1, choices=[0, 1])
    p.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    p.add_argument("--dp_buckets", type=int, default=1,
                   help="ZeRO-1 buckets; >1 reduces each bucket beside backward as soon as its gradients are written")
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--synthetic", action="store_true")
    p.add_argument("--n_layer", type=int, default=0, help="override the preset depth (smoke tests)")
    p.add_argument("--n_embd", type=int, default=0, help="override the preset width (smoke tests, small experiments)")
    p.add_argument("--n_head", type=int, default=0, help="override the number of attention heads")
    p.add_argument("--n_kv_head", type=int, default=0, help="override the number of key / value heads (LLaMA-3)")
    p.add_argument("--ffn_dim", type=int, default=0, help="override the SwiGLU width (LLaMA-3)")
    p.add_argument("--vocab_size", type=int, default=0, help="override the vocabulary size (synthetic data only)")
    p.add_argument("--save", default="", help="checkpoint directory to write at the end (and every --save_every steps)")
    p.add_argument("--save_every", type=int, default=0, help="also checkpoint every N optimizer steps (0 = only at the end)")
    p.add_argument("--resume", default="", help="checkpoint directory to resume from; 'auto' = the --save directory if it "
                                                "holds a checkpoint (restart-after-failure recipe: same command line again)")
    p.add_argument("--log_jsonl", default="")
    p.add_argument("--cuda_graph", action="store_true", help="capture the single-GPU training step in a CUDA graph")
    return p


def _config(family: str, args):
    import dataclasses

    from .models import GPT2_PRESETS, LLAMA3_PRESETS

    cfg = (GPT2_PRESETS if family == "gpt2" else LLAMA3_PRESETS)[args.model]
    cfg = dataclasses.replace(cfg)
    if args.n_layer:
        cfg.n_layer = args.n_layer
    for name in ("n_embd", "n_head", "n_kv_head", "ffn_dim"):
        if getattr(args, name) and hasattr(cfg, name):
            setattr(cfg, name, getattr(args, name))
    if args.vocab_size:
        cfg.vocab_size = args.vocab_size
        if hasattr(cfg, "padded_vocab_size"):
            cfg.padded_vocab_size = (args.vocab_size + 127) // 128 * 128
    cfg.block_size = max(args.sequence_length, min(cfg.block_size, 8192))
    return cfg


def _data(args, cfg, rank_dp: int, world_dp: int, pin: bool, drop_last: bool = False):
    from . import data

    if args.input_bin and not args.synthetic:
        ds = data.TinyShakespeareDataset(args.input_bin, args.sequence_length)
    else:
        n = max(64, args.batch_size * world_dp * 8)
        ds = data.SyntheticDataset(args.seed, cfg.vocab_size, args.sequence_length, n)
    return data.DataLoader(ds, args.batch_size, pin_memory=pin, rank=rank_dp, world=world_dp, drop_last=drop_last)


def train_main(family: str, argv=None) -> int:
    args = build_parser(family).parse_args(argv)
    import torch.distributed as dist

    import tinyinfinitrain_b200 as tit
    from .models import GPT2, LLaMA3
    from .utils import CudaTimer, JsonlLogger, ThroughputMeter, load_checkpoint, save_checkpoint

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = args.device == "cuda"
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if cuda:
        torch.cuda.set_device(local)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    cfg = _config(family, args)
    tp, pp = args.tensor_parallel, args.pipeline_parallel
    log = JsonlLogger(args.log_jsonl if rank == 0 else None)
    B, T = args.batch_size, args.sequence_length
    if args.resume == "auto":
        args.resume = args.save if args.save and os.path.exists(os.path.join(args.save, "meta.json")) else ""

    def lr_at(step: int) -> float:
        from .optim.schedule import warmup_cosine

        if not args.lr_decay_steps and not args.warmup_steps:
            return args.learning_rate
        return warmup_cosine(step, args.learning_rate, args.warmup_steps, args.lr_decay_steps or (1 << 62),
                             args.min_lr_ratio if args.lr_decay_steps else 1.0)

    def apply_lr(opt, step: int) -> float:
        lr = lr_at(step)
        if hasattr(opt, "set_lr"):
            opt.set_lr(lr)
        else:
            opt.lr = lr
        return lr

    if not distributed:
        # ------------------------------------------------------------------ one process
        cls = GPT2 if family == "gpt2" else LLaMA3
        model = cls.FromLLMC(args.llmc_filepath, device=dev, dtype=dtype) if args.llmc_filepath else \
            cls(cfg, device=dev, dtype=dtype, seed=args.seed)
        if args.optimizer == "sgd":
            opt = tit.optim.SGD(model.parameters(), args.learning_rate)
        else:
            opt = tit.optim.MixedPrecisionAdam(model.parameters(), lr=args.learning_rate, weight_decay=args.weight_decay,
                                               max_grad_norm=args.max_grad_norm)
        start = load_checkpoint(args.resume, model, opt) if args.resume else 0
        loader = _data(args, cfg, 0, 1, cuda)
        accum = max(1, args.total_batch_size // (B * T)) if args.total_batch_size else 1
        meter = ThroughputMeter(B * T * accum, model.flops_per_token(T), 1398.5 if cuda else 0.0)
        tok = tit.data.Tokenizer(args.tokenizer_bin) if args.tokenizer_bin else None
        it = start * accum                       # a resumed run continues with the batches the first run had not seen
        for step in range(start, args.num_iteration):
            lr = apply_lr(opt, step)
            with CudaTimer() as tm:
                opt.zero_grad()
                lossf = 0.0
                for _ in range(accum):
                    x, y = loader.batch(it % len(loader))
                    it += 1
                    x, y = x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)
                    fused = cuda and dtype == torch.bfloat16
                    _, loss = model(x, y, return_logits=not fused)
                    (loss / accum).backward()
                    lossf += float(loss) / accum
                opt.step()
            rep = meter.report(tm.ms)
            if rank == 0:
                print(f"step {step + 1}/{args.num_iteration} | loss {lossf:.6f} | lr {lr:.2e} | "
                      f"{tm.ms:.2f} ms | {rep['tokens_per_s']:.0f} tok/s" + (f" | mfu {rep['mfu']:.3f}" if 'mfu' in rep else ""),
                      flush=True)
            log.log(step=step + 1, loss=lossf, lr=lr, **rep)
            if tok is not None and args.freq_generate_txt and (step + 1) % args.freq_generate_txt == 0:
                tok.GenerateText(model, B, T, args.text_length, dev, stream=sys.stdout)
            if args.save and args.save_every and (step + 1) % args.save_every == 0 and step + 1 < args.num_iteration:
                save_checkpoint(args.save, model, opt, step + 1)
        if args.save:
            save_checkpoint(args.save, model, opt, args.num_iteration)
        log.close()
        return 0

    # ---------------------------------------------------------------------- dp x pp x tp
    from .utils import ParallelTrainStep

    nm = max(1, args.num_microbatches)
    sd = None
    if args.llmc_filepath:
        from .utils.llmc import map_checkpoint

        # memory-mapped views: every rank touches only the rows / columns of its own shard
        fam, _, sd = map_checkpoint(args.llmc_filepath)
        assert fam == family, f"{args.llmc_filepath} is a {fam} checkpoint"
    pstep = ParallelTrainStep(cfg, B, T, dev, dtype, tp=tp, pp=pp, num_microbatches=nm, zero_stage=args.zero_stage,
                              comm=args.comm, dp_buckets=args.dp_buckets, lr=args.learning_rate,
                              weight_decay=args.weight_decay, max_grad_norm=args.max_grad_norm, seed=args.seed,
                              full_state_dict=sd)
    mesh, model, opt = pstep.mesh, pstep.model, pstep.opt
    # every rank keeps its own optimizer shard (fp32 master weights, moments, step); on resume the data-parallel
    # group rebuilds the parameters from the master shards
    layout = {"tp": tp, "pp": pp, "dp": mesh.dp}
    start = load_checkpoint(args.resume, model, opt, rank=rank, world=world, layout=layout) if args.resume else 0
    # static shapes (pipeline receive buffers, token shards): the incomplete last batch is dropped, and every
    # data-parallel rank sees the same number of batches
    loader = _data(args, cfg, mesh.dp_rank, mesh.dp, cuda, drop_last=True)
    meter = ThroughputMeter(pstep.tokens_per_step, 0.0, 0.0)
    it = start * nm
    for step in range(start, args.num_iteration):
        lr = apply_lr(opt, step)
        # device-timed (CUDA events on the launching stream; wall clock only on the CPU path), max over ranks
        with CudaTimer() as tm:
            host = []
            for _ in range(nm):
                host.append(loader.batch(it % len(loader)))
                it += 1
            hl = pstep(host)
        ms = torch.tensor([tm.ms], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        lossv = pstep.loss.detach().reshape(1).clone()
        dist.all_reduce(lossv)
        lossv = lossv.item() / (mesh.dp * tp)          # the last stage of every replica (and each tp rank) reports it
        rep = meter.report(ms.item())
        if rank == 0:
            mem = f" | peak mem {torch.cuda.max_memory_allocated(dev) / 2**30:.1f} GiB" if cuda else ""
            print(f"step {step + 1}/{args.num_iteration} | loss {lossv:.6f} | lr {lr:.2e} | "
                  f"{ms.item():.2f} ms | {rep['tokens_per_s']:.0f} tok/s | tp{tp} pp{pp} dp{mesh.dp}{mem}", flush=True)
        log.log(step=step + 1, loss=lossv, lr=lr, **rep)
        if args.save and args.save_every and (step + 1) % args.save_every == 0 and step + 1 < args.num_iteration:
            save_checkpoint(args.save, model, opt, step + 1, rank=rank, world=world, extra=layout, mesh=mesh)
            dist.barrier()
    if args.save:
        save_checkpoint(args.save, model, opt, args.num_iteration, rank=rank, world=world, extra=layout, mesh=mesh)
        dist.barrier()
    if cuda:
        status = tit._lib.C.status_read(True)
        if status:
            print(f"rank {rank}: kernel status word {status} (a bounded device-side wait gave up)", file=sys.stderr)
    log.close()
    dist.destroy_process_group()
    return 0
