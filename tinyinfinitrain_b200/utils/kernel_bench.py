"""Single-kernel benchmark driver: times one kernel of the library on one shape with CUDA events
and reports achieved throughput against the measured peaks (``MEASURED_PEAKS.json`` at the
repository root when present, otherwise the documented fallback).  The same command line is what
the ncu captures summarised under ``profiles/`` run.

    python -m tinyinfinitrain_b200.utils.kernel_bench gemm --m 8192 --n 3072 --k 768
    python -m tinyinfinitrain_b200.utils.kernel_bench attn_bwd --b 8 --t 1024 --h 12 --hd 64

The fused compute+collective kernels can be run on ONE GPU for profiling: ``ag_gemm`` and
``rs_adam`` take ``--world W`` and treat W local buffers as the peers (every load and store a
rank would send over NVLink goes to local memory instead, the instruction stream is the one the
multi-GPU run executes; ``rs_adam`` uses plain peer loads/stores, not multimem);
``gemm_rs`` runs as a group of one rank (its own partial tiles are the only ones it waits for);
``param_gather_gemm`` pulls the weight rows of ``--world`` owners from local copies.
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters, warmup=3, flush=None):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    tot = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()          # > L2 so the timed launch starts cold
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        e1.synchronize()
        tot += e0.elapsed_time(e1)
    return tot / iters


def gemm_sweep(C, model: str, iters: int):
    """Every GEMM of one transformer layer (forward, dgrad, wgrad) plus the vocabulary projection, this library against
    torch.matmul (cuBLAS) on the same tensors: `iters` launches back to back between two CUDA events, no L2 flush
    (inside a training step the operands of a GEMM were just written by the kernel before it)."""
    dev, bf = "cuda", torch.bfloat16
    hbm, tflops, src = peaks()
    if model == "gpt2":
        M, shapes = 8192, [("c_attn", 2304, 768), ("attn.c_proj", 768, 768), ("c_fc", 3072, 768), ("mlp.c_proj", 768, 3072),
                           ("lm_head", 50304, 768)]
    elif model == "gpt2xl":
        M, shapes = 4096, [("c_attn", 4800, 1600), ("attn.c_proj", 1600, 1600), ("c_fc", 6400, 1600), ("mlp.c_proj", 1600, 6400)]
    else:  # llama-1B
        M, shapes = 8192, [("c_attn", 3072, 2048), ("attn.c_proj", 2048, 2048), ("c_fc", 16384, 2048), ("mlp.c_proj", 2048, 8192)]

    def run(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        e1.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3   # us

    rows = []
    for name, N, K in shapes:
        X = torch.randn(M, K, device=dev).to(bf)          # activations
        W = (torch.randn(N, K, device=dev) * 0.02).to(bf)  # weight [out, in]
        dY = torch.randn(M, N, device=dev).to(bf)
        dWf = torch.zeros(N, K, device=dev)
        Wt = W.t().contiguous()
        cases = [
            ("fwd   Y=X.W^T", lambda: C.gemm(X, W), lambda: torch.matmul(X, W.t())),
            ("dgrad dX=dY.W", lambda: C.gemm(dY, W, False, True), lambda: torch.matmul(dY, W)),
            ("wgrad dW+=dY^T.X (fp32 out)", lambda: C.gemm(dY, X, True, True, out=dWf, accumulate=True),
             lambda: torch.matmul(dY.t(), X)),
        ]
        pair_cases = [lambda: C.gemm(X, W, tile_n=512), lambda: C.gemm(dY, W, False, True, tile_n=512),
                      lambda: C.gemm(dY, X, True, True, out=dWf, accumulate=True, tile_n=512)]
        for (label, ours, lib), pair in zip(cases, pair_cases):
            t_o, t_l, t_p = run(ours), run(lib), run(pair)
            fl = 2.0 * M * N * K
            rows.append({"layer": name, "case": label, "M": M, "N": N, "K": K, "ours_us": t_o, "torch_us": t_l,
                         "pair_us": t_p,   # forced CTA pairs (256 x 256 tiles), whatever the planner would pick
                         "ours_frac_of_bf16_peak": fl / t_o / 1e6 / tflops, "ours_over_torch": t_l / t_o})
        del X, W, dY, dWf, Wt
    print(f"{'layer':<12} {'case':<30} {'N':>6} {'K':>6} {'ours us':>9} {'torch us':>9} {'frac peak':>9} {'speedup':>8} {'pairs us':>9}")
    for r in rows:
        print(f"{r['layer']:<12} {r['case']:<30} {r['N']:>6} {r['K']:>6} {r['ours_us']:>9.1f} {r['torch_us']:>9.1f} "
              f"{r['ours_frac_of_bf16_peak']:>9.3f} {r['ours_over_torch']:>8.2f} {r['pair_us']:>9.1f}")
    print(json.dumps({"kernel": "gemm_sweep", "model": model, "peaks": src, "status": int(C.status_read(True)), "rows": rows}))


def main():
    from .._lib import C
    from .. import ops

    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "gemm_nt", "gemm_wgrad", "attn_fwd", "attn_bwd", "layernorm_fwd", "layernorm_bwd",
                                       "xent", "adam", "gelu_gemm", "ag_gemm", "gemm_rs", "rs_adam", "clip", "embedding_bwd",
                                       "reduce", "transpose_view", "colsum", "param_gather_gemm", "gemm_sweep"])
    ap.add_argument("--model", default="gpt2", choices=["gpt2", "gpt2xl", "llama1b"], help="gemm_sweep: whose layer shapes")
    ap.add_argument("--deterministic", action="store_true", help="embedding_bwd: sorted segment reduction instead of atomics")
    ap.add_argument("--world", type=int, default=4)
    ap.add_argument("--helpers", type=int, default=0, help="ag_gemm: copying CTAs (0: sized by the launcher)")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=3072)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--b", type=int, default=8)
    ap.add_argument("--t", type=int, default=1024)
    ap.add_argument("--h", type=int, default=12)
    ap.add_argument("--hkv", type=int, default=0)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--tile_n", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--no_flush", action="store_true")
    ap.add_argument("--residual", action="store_true", help="layernorm_bwd: add a residual gradient to dx")
    a = ap.parse_args()
    if a.kernel == "gemm_sweep":
        return gemm_sweep(C, a.model, a.iters)
    dev = "cuda"
    hbm, tflops, src = peaks()
    flush = None if a.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    bf = torch.bfloat16
    flops = bytes_ = 0.0
    if a.kernel in ("gemm", "gemm_nt", "gemm_wgrad", "gelu_gemm"):
        M, N, K = a.m, a.n, a.k
        flops = 2.0 * M * N * K
        bytes_ = 2.0 * (M * K + N * K + M * N)
        if a.kernel == "gemm":
            A, B = torch.randn(M, K, device=dev).to(bf), torch.randn(N, K, device=dev).to(bf)
            fn = lambda: C.gemm(A, B, tile_n=a.tile_n)
        elif a.kernel == "gelu_gemm":
            A, B = torch.randn(M, K, device=dev).to(bf), torch.randn(N, K, device=dev).to(bf)
            bias = torch.randn(N, device=dev).to(bf)
            fn = lambda: C.gemm(A, B, epilogue=2, bias=bias, want_aux_out=True, tile_n=a.tile_n)
        elif a.kernel == "gemm_nt":   # dgrad: dY [M, K] . W [K, N]
            A, B = torch.randn(M, K, device=dev).to(bf), torch.randn(K, N, device=dev).to(bf)
            fn = lambda: C.gemm(A, B, False, True, tile_n=a.tile_n)
        else:                          # wgrad: dY^T [M=out, K=tokens] X [tokens, N]
            A, B = torch.randn(K, M, device=dev).to(bf), torch.randn(K, N, device=dev).to(bf)
            out = torch.zeros(M, N, device=dev)
            fn = lambda: C.gemm(A, B, True, True, out=out, accumulate=True, tile_n=a.tile_n)
    elif a.kernel in ("attn_fwd", "attn_bwd"):
        Hkv = a.hkv or a.h
        W = (a.h + 2 * Hkv) * a.hd
        qkv = (torch.randn(a.b, a.t, W, device=dev) * 0.5).to(bf)
        q = qkv[..., :a.h * a.hd].view(a.b, a.t, a.h, a.hd)
        k = qkv[..., a.h * a.hd:(a.h + Hkv) * a.hd].view(a.b, a.t, Hkv, a.hd)
        v = qkv[..., (a.h + Hkv) * a.hd:].view(a.b, a.t, Hkv, a.hd)
        scale = a.hd ** -0.5
        fwd_flops = 4.0 * a.b * a.h * a.t * a.t * a.hd / 2
        if a.kernel == "attn_fwd":
            flops = fwd_flops
            fn = lambda: C.attn_fwd(q, k, v, scale)
        else:
            o, lse = C.attn_fwd(q, k, v, scale)
            do = torch.randn_like(o)
            flops = 2.5 * fwd_flops
            fn = lambda: C.attn_bwd(do, q, k, v, o, lse, scale)
        bytes_ = 2.0 * qkv.numel() * 2
    elif a.kernel in ("layernorm_fwd", "layernorm_bwd"):
        x = torch.randn(a.m, a.k, device=dev).to(bf)
        w, b = torch.ones(a.k, device=dev).to(bf), torch.zeros(a.k, device=dev).to(bf)
        if a.kernel == "layernorm_fwd":
            bytes_ = 2.0 * x.numel() * 2
            fn = lambda: C.layernorm_fwd(x, w, b, 1e-5)
        else:
            y, mean, rstd = C.layernorm_fwd(x, w, b, 1e-5)
            dy = torch.randn_like(x)
            bytes_ = (4.0 if a.residual else 3.0) * x.numel() * 2
            dres = torch.randn_like(x) if a.residual else None
            fn = lambda: C.layernorm_bwd(dy, x, w, mean, rstd, dres=dres)
    elif a.kernel == "ag_gemm":
        # X = concat of W shards [M/W, K]; Y = X . B^T, B [N, K]
        M, N, K, W = a.m, a.n, a.k, a.world
        shards = [torch.randn(M // W, K, device=dev).to(bf) for _ in range(W)]
        B = torch.randn(N, K, device=dev).to(bf)
        flops = 2.0 * M * N * K
        bytes_ = 2.0 * (2 * M * K + N * K + M * N)
        ptrs = [t.data_ptr() for t in shards]
        fn = lambda: C.gemm_ag(ptrs, 0, M // W, K, B, False, 0, None, False, max(a.helpers, 0))
    elif a.kernel == "param_gather_gemm":
        # Y = X . W^T with the rows of W owned by W ranks: `world` local copies stand in for the ranks' memory
        M, N, K, W = a.m, a.n, a.k, a.world
        X = torch.randn(M, K, device=dev).to(bf)
        copies = [(torch.randn(N, K, device=dev) * 0.1).to(bf) for _ in range(W)]
        npr = N // W
        ptrs = [copies[r].data_ptr() + r * npr * K * 2 for r in range(W)]
        flops = 2.0 * M * N * K
        bytes_ = 2.0 * (M * K + 2 * N * K + M * N)
        fn = lambda: C.gemm_param_gather(X, copies[0], ptrs, 0, helper_ctas=max(a.helpers, 0))
    elif a.kernel == "gemm_rs":
        M, N, K = a.m, a.n, a.k
        A, B = torch.randn(M, K, device=dev).to(bf), torch.randn(N, K, device=dev).to(bf)
        recv = torch.empty(M, N, device=dev, dtype=bf)
        cnt = torch.zeros(max(128, M // 128 + 1), device=dev, dtype=torch.int32)
        flops = 2.0 * M * N * K
        bytes_ = 2.0 * (M * K + N * K + 3 * M * N)
        fn = lambda: C.gemm_rs(A, B, False, [recv.data_ptr()], [cnt.data_ptr()], 0, None, None,
                               min(a.helpers or 8, M // 128))
    elif a.kernel == "rs_adam":
        n, W = a.m * a.n, a.world
        n -= n % (8 * W * 16)
        S = n // W
        grads = [torch.randn(n, device=dev) for _ in range(W)]
        params = [torch.empty(n, device=dev, dtype=bf) for _ in range(W)]
        master, m, v = torch.randn(S, device=dev), torch.zeros(S, device=dev), torch.zeros(S, device=dev)
        # per launch: W gradient shards read, fp32 state read + written, W bf16 parameter shards written
        bytes_ = S * (4.0 * W + 3 * 4 * 2 + 2.0 * W)
        gp, pp = [t.data_ptr() for t in grads], [t.data_ptr() for t in params]
        fn = lambda: C.rs_adam_ag(gp, pp, 0, 0, master, m, v, 0, 0, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, 1.0 / W)
    elif a.kernel == "clip":
        n = a.m * a.n
        g = torch.randn(n, device=dev) * 0.01
        out2 = torch.zeros(2, device=dev)
        bytes_ = n * 4.0 * 3            # norm pass reads once; the scaling pass reads and writes (max_norm tiny: always clips)
        fn = lambda: C.clip_grad_norm_(g, 1e-6, 1.0, out2)
    elif a.kernel == "embedding_bwd":
        idx = torch.randint(0, a.n, (a.b, a.t), device=dev)
        dout = torch.randn(a.b, a.t, a.k, device=dev).to(bf)
        dw = torch.zeros(a.n, a.k, device=dev)
        bytes_ = a.b * a.t * a.k * (2.0 + 8.0)   # gradient rows read, fp32 table rows read-modify-written
        fn = lambda: C.embedding_bwd(idx, dout, dw, None, 0, a.n, a.deterministic)
    elif a.kernel == "reduce":
        x = torch.randn(a.m, a.k, device=dev).to(bf)
        bytes_ = x.numel() * 2.0
        fn = lambda: C.reduce_dim(x, 0, 1, False)          # row sums
    elif a.kernel == "transpose_view":
        x = torch.randn(a.b, a.t, a.h, a.hd, device=dev).to(bf)
        v = x.transpose(1, 2)                              # [B, H, T, hd] view materialised by the gather kernel
        bytes_ = x.numel() * 4.0
        fn = lambda: C.gather_view(x, list(v.shape), list(v.stride()), 0)
    elif a.kernel == "colsum":
        x = torch.randn(a.m, a.n, device=dev).to(bf)
        outc = torch.zeros(a.n, device=dev)
        bytes_ = x.numel() * 2.0
        fn = lambda: C.colsum(x, outc, False)
    elif a.kernel == "xent":
        logits = torch.randn(a.m, a.n, device=dev).to(bf)
        tgt = torch.randint(0, a.n - 47, (a.m,), device=dev)
        bytes_ = 2.0 * logits.numel() * 2
        fn = lambda: C.xent_fused(logits, tgt, a.n - 47, 1.0 / a.m, True, 1.0 / a.m)
    else:
        n = a.m * a.n
        w, g = torch.randn(n, device=dev), torch.randn(n, device=dev)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        lp = torch.empty(n, device=dev, dtype=bf)
        bytes_ = n * (4 * 4 + 3 * 4 + 2)
        fn = lambda: C.adam_flat(w, lp, g, m, v, 1e-3, 0.9, 0.999, 1e-8, 0.0, 1, 1.0)
    ms = timeit(fn, a.iters, flush=flush)
    torch.cuda.synchronize()
    out = {"kernel": a.kernel, "ms": ms, "status": int(C.status_read(True)), "peaks": src}
    if flops:
        out["tflops"] = flops / ms / 1e9
        out["frac_of_bf16_peak"] = out["tflops"] / tflops
    if bytes_:
        out["gbs"] = bytes_ / ms / 1e6
        out["frac_of_hbm_peak"] = out["gbs"] / hbm
    out["args"] = {k: v for k, v in vars(a).items() if k != "kernel"}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
