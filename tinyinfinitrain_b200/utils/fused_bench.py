"""Multi-GPU micro-benchmark of the fused compute+collective kernels against their unfused
NCCL + tcgen05 baselines (run under torchrun, one rank per GPU).

    torchrun --nproc-per-node 8 -m tinyinfinitrain_b200.utils.fused_bench

For each case the time is device-side (CUDA events), the maximum over ranks, averaged over
``--iters`` launches after warm-up; the roofline is the slower of (FLOPs / measured bf16 GEMM peak)
and (bytes one GPU must send or receive over NVLink / 770 GB/s, the measured peer-copy bandwidth).
Rank 0 prints one JSON line per case.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def _time(fn, iters, warmup=3):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main():
    from .kernel_bench import peaks
    from ..parallel.tp import TPComm
    from ..parallel.zero import DistributedOptimizer

    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=8192, help="B*T of the tensor-parallel cases")
    ap.add_argument("--d_model", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--params_m", type=int, default=124, help="millions of parameters of the ZeRO-1 case")
    ap.add_argument("--json_out", default="", help="file that receives all records as a JSON list")
    a = ap.parse_args()
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    _, tflops, src = peaks()
    nccl, fused = TPComm(dist.group.WORLD, "nccl"), TPComm(dist.group.WORLD, "fused")
    M, Cd, F = a.tokens, a.d_model, a.ffn
    Ms = M // world
    out = []

    def report(name, ms_f, ms_n, flops, link_bytes):
        t_comp = flops / (tflops * 1e12) * 1e3
        t_link = link_bytes / (NVLINK_GBS * 1e9) * 1e3
        roof = max(t_comp, t_link)
        rec = {"case": name, "world": world, "fused_ms": ms_f, "nccl_unfused_ms": ms_n, "speedup": ms_n / ms_f,
               "roofline_ms": roof, "bound": "compute" if t_comp >= t_link else "nvlink",
               "fused_frac_of_roofline": roof / ms_f, "peaks": src}
        out.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)

    g = torch.Generator(device=dev).manual_seed(rank)
    # F1: all-gather -> GEMM (column parallel: QKV-like [C -> 3C/world... use FFN up 2F/world])
    x_s = (torch.randn(Ms, Cd, device=dev, generator=g) * 0.5).bfloat16()
    for name, N in (("ag_gemm_ffn_up", 2 * F // world), ("ag_gemm_qkv", 3 * Cd // world)):
        w = (torch.randn(N, Cd, device=dev, generator=g) * 0.05).bfloat16()
        ms_f = _time(lambda: fused.ag_gemm(x_s, w), a.iters)
        ms_n = _time(lambda: nccl.ag_gemm(x_s, w), a.iters)
        report(name, ms_f, ms_n, 2.0 * M * N * Cd, (world - 1) * Ms * Cd * 2)
    # F2: GEMM -> reduce-scatter (row parallel: FFN down [F/world -> C], attention out [C/world -> C])
    for name, K in (("gemm_rs_ffn_down", F // world), ("gemm_rs_attn_out", Cd // world)):
        y = (torch.randn(M, K, device=dev, generator=g) * 0.5).bfloat16()
        w = (torch.randn(Cd, K, device=dev, generator=g) * 0.05).bfloat16()
        ms_f = _time(lambda: fused.gemm_rs(y, w), a.iters)
        ms_n = _time(lambda: nccl.gemm_rs(y, w), a.iters)
        report(name, ms_f, ms_n, 2.0 * M * Cd * K, (world - 1) * Ms * Cd * 2)
    # F3: gradient reduce-scatter + Adam + parameter all-gather
    n = a.params_m * 1000 * 1000
    res = {}
    for comm in ("fused", "nccl"):
        p = torch.nn.Parameter(torch.zeros(n, device=dev, dtype=torch.bfloat16))
        opt = DistributedOptimizer([p], lr=1e-4, comm=comm)
        opt.flat.grad.normal_()

        def step():
            for q in opt.params:
                q._fresh_grad = False
            opt.step()

        res[comm] = _time(step, a.iters)
        del opt, p
        torch.cuda.empty_cache()
    link = (world - 1) / world * n * 4 + (world - 1) / world * n * 2   # fp32 gradient shards in, bf16 parameter shards out
    report(f"rs_adam_ag_{a.params_m}M", res["fused"], res["nccl"], 0.0, link)
    # F4: parameter all-gather -> GEMM (weight rows sharded over the ranks) against NCCL all-gather + GEMM
    from .._lib import C
    from ..parallel.param_gather import GatheredWeightLinear

    for name, (N, K) in (("param_gather_gemm_ffn_up", (F, Cd)), ("param_gather_gemm_attn_out", (Cd, Cd))):
        if N % (128 * world):
            continue
        layer = GatheredWeightLinear(K, N, bias=False, device=dev)
        xin = (torch.randn(M, K, device=dev, generator=g) * 0.5).bfloat16()
        mine = layer.weight.detach()[layer.own_rows()].clone()
        full = torch.empty(N, K, device=dev, dtype=torch.bfloat16)

        def fused_step():
            layer.barrier()
            C.gemm_param_gather(xin, layer.weight.detach(), layer.peer_row_ptrs, layer.rank, helper_ctas=layer.helper_ctas)

        def nccl_step():
            dist.all_gather_into_tensor(full, mine)
            C.gemm(xin, full)

        ms_f, ms_n = _time(fused_step, a.iters), _time(nccl_step, a.iters)
        report(name, ms_f, ms_n, 2.0 * M * N * K, (world - 1) / world * N * K * 2)
        del layer
    # standalone all-reduce on symmetric memory against NCCL (fp32, the size of a GPT-2 124M gradient buffer)
    from ..parallel.collectives import SymmCollective

    coll = SymmCollective(n, torch.float32, dev)
    coll.tensor.normal_()
    plain = coll.tensor.clone()
    ms_f = _time(lambda: coll.all_reduce_(), a.iters)
    ms_n = _time(lambda: dist.all_reduce(plain), a.iters)
    report(f"allreduce_fp32_{a.params_m}M", ms_f, ms_n, 0.0, 2.0 * (world - 1) / world * n * 4)
    if rank == 0 and a.json_out:
        json.dump(out, open(a.json_out, "w"), indent=1)
    st = C.status_read(True)
    if st:
        print(f"rank {rank}: status {st}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
