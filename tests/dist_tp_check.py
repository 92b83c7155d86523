"""Worker for the multi-GPU tensor-parallel test (torchrun, one rank per GPU).

1. all-gather -> GEMM and GEMM -> reduce-scatter fused kernels against NCCL + tcgen05 GEMM and
   against fp32 PyTorch math, several shapes, repeated calls (buffer reuse).
2. A sequence-parallel LLaMA-3 and GPT-2 block stack: fused vs NCCL path, loss and gradients.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import tinyinfinitrain_b200 as tit
    from tinyinfinitrain_b200.models import GPT2, GPT2Config, LLaMA3, LLaMA3Config
    from tinyinfinitrain_b200.models.tp_models import TPTransformer
    from tinyinfinitrain_b200.parallel.tp import TPComm, sync_sequence_parallel_grads

    nccl = TPComm(dist.group.WORLD, "nccl")
    fused = TPComm(dist.group.WORLD, "fused")
    ok = True
    msgs = []
    for rep in range(2):
        if rep == 1:
            # poison, then verify: every staging / receive buffer of the fused kernels is filled with NaN (the arrival
            # counters are left alone), so a tile that a kernel reads before its producer has written it cannot
            # pass unnoticed in the second round
            ft = fused._fused
            torch.cuda.synchronize()
            dist.barrier()
            for buf in ft._ag.values():
                buf.tensor.fill_(float("nan"))
            for recv, _cnt in ft._rs.values():
                recv.tensor.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            ft.new_step()
        for (Ms, K, N) in [(128, 256, 512), (256, 2048, 384), (1024, 512, 1024)]:
            g = torch.Generator(device=dev).manual_seed(100 + rank + rep)
            x_s = (torch.randn(Ms, K, device=dev, generator=g) * 0.5).bfloat16()
            gw = torch.Generator(device=dev).manual_seed(7 + rank)
            w = (torch.randn(N, K, device=dev, generator=gw) * 0.1).bfloat16()
            b = (torch.randn(N, device=dev, generator=gw) * 0.1).bfloat16()
            y0, X0 = nccl.ag_gemm(x_s, w, b)
            y1, X1 = fused.ag_gemm(x_s, w, b)
            e_ag = (y0.float() - y1.float()).abs().max().item()
            e_x = (X0.float() - X1.float()).abs().max().item()
            ref = X0.float() @ w.float().t() + b.float()
            e_ref = (y1.float() - ref).abs().max().item()
            # row parallel: y [M, K] local features, weight [N, K]
            M = Ms * world
            yin = (torch.randn(M, K, device=dev, generator=g) * 0.5).bfloat16()
            res = torch.randn(Ms, N, device=dev, generator=g).bfloat16()
            z0 = nccl.gemm_rs(yin, w, False, b, res)
            z1 = fused.gemm_rs(yin, w, False, b, res)
            # partial sums grow with the group size, and so does one bf16 ulp of the result: compare relative to the
            # largest element
            e_rs = ((z0.float() - z1.float()).abs().max() / z0.float().abs().max()).item()
            wt = w.t().contiguous()  # MN-major weight path (dgrad form)
            z2 = fused.gemm_rs(yin, wt, True)
            z3 = nccl.gemm_rs(yin, wt, True)
            e_rs2 = ((z2.float() - z3.float()).abs().max() / z3.float().abs().max()).item()
            torch.cuda.synchronize()
            good = e_ag < 5e-2 and e_x == 0.0 and e_ref < 0.15 and e_rs < 4e-2 and e_rs2 < 4e-2
            ok = ok and good
            msgs.append(f"[{Ms},{K},{N}] ag {e_ag:.3g} X {e_x:.3g} ref {e_ref:.3g} rs {e_rs:.3g} rs_mn {e_rs2:.3g}")
    status = tit._lib.C.status_read(True)
    ok = ok and status == 0

    # model level
    for cfg in (LLaMA3Config(block_size=256, vocab_size=1000, n_layer=2, n_head=8, n_kv_head=8 if world > 2 else 2,
                             n_embd=512, ffn_dim=1024),
                GPT2Config(block_size=256, vocab_size=1000, n_layer=2, n_head=8, n_embd=512)):
        gi = torch.Generator().manual_seed(5)
        idx = torch.randint(0, 1000, (4, 256), generator=gi).to(dev)
        tgt = torch.roll(idx, -1, 1)
        res = {}
        for name, comm in (("nccl", nccl), ("fused", fused)):
            model = TPTransformer(cfg, comm, device=dev, dtype=torch.bfloat16, seed=42)
            loss = model(idx, tgt)
            loss.backward()
            sync_sequence_parallel_grads(model.parameters(), comm)
            res[name] = (loss.item(), {n: p.grad.float().clone() for n, p in model.named_parameters() if p.grad is not None})
        dl = abs(res["nccl"][0] - res["fused"][0])
        worst = 0.0
        for n, gn in res["nccl"][1].items():
            gf = res["fused"][1][n]
            worst = max(worst, ((gn - gf).abs().max() / (gn.abs().max() + 1e-6)).item())
        # the same seed gives every rank exactly its slices of the single-GPU model: the losses must agree
        single = (LLaMA3 if isinstance(cfg, LLaMA3Config) else GPT2)(cfg, device=dev, dtype=torch.bfloat16, seed=42)
        l1 = single(idx, tgt, return_logits=False)[1].item()
        good = dl < 2e-2 and worst < 8e-2 and abs(l1 - res["fused"][0]) < 3e-2
        ok = ok and good
        msgs.append(f"{type(cfg).__name__}: loss nccl {res['nccl'][0]:.4f} fused {res['fused'][0]:.4f} single-GPU {l1:.4f} "
                    f"worst rel grad diff {worst:.3g}")
    status = tit._lib.C.status_read(True)
    ok = ok and status == 0
    print(f"rank {rank}: ok={ok} status={status}\n  " + "\n  ".join(msgs), flush=True)
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    dist.destroy_process_group()
    sys.exit(0 if t.item() == 1.0 else 1)


if __name__ == "__main__":
    main()
