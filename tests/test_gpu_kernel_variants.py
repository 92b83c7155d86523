"""GPU numerics of the single-GPU kernels beyond the core training set: norm backward with the residual gradient folded in, the attention pipelines
on long and ragged sequences, column sums, 128x192 GEMM tiles, gradient clipping,
deterministic embedding gradient, one-GPU runs of the symmetric-memory collectives and the parameter-gather GEMM,
vocabulary-parallel cross entropy, reductions and view kernels.  Each is compared against plain PyTorch fp32 math of
the same op (or against the kernel it replaces)."""
import os
import subprocess
import sys

import pytest
import torch

from _launch import run_group
from tinyinfinitrain_b200 import ops
from tinyinfinitrain_b200._lib import C

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16
HERE = os.path.dirname(os.path.abspath(__file__))


def _status_ok():
    torch.cuda.synchronize()
    assert C.status_read(True) == 0



@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("rows,cols", [(8192, 768), (1000, 1024), (4737, 512), (37, 256), (5, 64), (300, 2048), (64, 4096)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_backward_with_residual_gradient(dtype, rows, cols, rms):
    """Fewer rows than warps, an odd row count (the second row of a warp's last pair is missing), widths served by
    the two-rows-in-flight kernel (3 and 4 vectors per lane), by the one-row-per-warp kernel (8) and by the
    CTA-per-row kernel; every one has to add `dres` to dx inside the kernel and give the same bits on every run."""
    torch.manual_seed(19)
    x = (torch.randn(rows, cols, device=DEV) * 1.5 + 0.3).to(dtype)
    w = (torch.rand(cols, device=DEV) + 0.5).to(dtype)
    b = torch.randn(cols, device=DEV).to(dtype)
    dy = torch.randn(rows, cols, device=DEV).to(dtype)
    dres = torch.randn(rows, cols, device=DEV).to(dtype)
    xr = x.float().requires_grad_(True)
    wr, br = w.float().requires_grad_(True), b.float().requires_grad_(True)
    if rms:
        y, rstd = C.rmsnorm_fwd(x, w, 1e-5)
        ref = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
        one = lambda **kw: C.rmsnorm_bwd(dy, x, w, rstd, **kw)
    else:
        y, mean, rstd = C.layernorm_fwd(x, w, b, 1e-5)
        ref = torch.nn.functional.layer_norm(xr, (cols,), wr, br, 1e-5)
        one = lambda **kw: C.layernorm_bwd(dy, x, w, mean, rstd, **kw)
    ref.backward(dy.float())
    runs = [one() for _ in range(3)]
    for r in runs[1:]:
        assert all(torch.equal(a, c) for a, c in zip(runs[0], r))              # fixed summation order
    tol_x = 3e-2 if dtype == BF else 2e-5
    tol_w = 4e-3 * rows ** 0.5 if dtype == BF else 2e-4 * rows ** 0.5
    assert torch.allclose(runs[0][0].float(), xr.grad, atol=tol_x, rtol=2e-2)
    assert torch.allclose(runs[0][1], wr.grad, atol=tol_w, rtol=1e-2)
    if not rms:
        assert torch.allclose(runs[0][2], br.grad, atol=tol_w, rtol=1e-2)
    # residual gradient folded into dx; weight gradients accumulated into given buffers
    dw_acc = torch.ones(cols, device=DEV)
    extra = {"dw": dw_acc, "accumulate": True, "dres": dres}
    if not rms:
        extra["db"] = torch.ones(cols, device=DEV)
    out = one(**extra)
    assert torch.allclose(out[0].float(), xr.grad + dres.float(), atol=2 * tol_x, rtol=2e-2)
    assert torch.allclose(dw_acc, 1.0 + wr.grad, atol=tol_w, rtol=1e-2)
    if not rms:
        assert torch.allclose(extra["db"], 1.0 + br.grad, atol=tol_w, rtol=1e-2)
    _status_ok()


def test_norm_fork_folds_the_residual_gradient(monkeypatch):
    """GPT-2 gradients with the residual gradient added inside the norm backward kernel (`fork`) equal the gradients
    of the same model when autograd sums the two branches with a separate add."""
    from tinyinfinitrain_b200.models import GPT2, GPT2Config
    from tinyinfinitrain_b200.ops import functional as Fn
    cfg = GPT2Config(block_size=64, vocab_size=300, padded_vocab_size=320, n_layer=2, n_head=2, n_embd=128)
    idx = torch.randint(0, 300, (2, 64), device=DEV)
    tgt = torch.randint(0, 300, (2, 64), device=DEV)
    grads = []
    for folded in (True, False):
        if not folded:
            monkeypatch.setattr(Fn, "layernorm_fork", lambda x, w, b, eps=1e-5, out=None: (Fn.layernorm(x, w, b, eps), x))
            monkeypatch.setattr(ops, "layernorm_fork", Fn.layernorm_fork, raising=False)
        model = GPT2(cfg, device=DEV, dtype=BF, seed=5)
        loss = model(idx, tgt)[1]
        loss.backward()
        grads.append({n: p.grad.float().clone() for n, p in model.named_parameters()})
    for n in grads[0]:
        scale = grads[0][n].abs().max().item() + 1e-6
        assert (grads[0][n] - grads[1][n]).abs().max().item() < 0.05 * scale, n
    _status_ok()


@pytest.mark.parametrize("M,N,K,world,helpers", [(1024, 512, 256, 4, 0), (2048, 3072, 768, 2, 0), (8192, 8192, 1024, 8, 0),
                                                  (4096, 2304, 768, 4, 8), (4096, 1024, 2048, 4, 40), (1024, 256, 320, 8, 3)])
def test_all_gather_gemm_with_local_shards_as_peers(M, N, K, world, helpers):
    """All-gather -> GEMM on one GPU: `world` local tensors stand in for the ranks' shards.  The copying CTAs move
    them with bulk copies through shared memory and then join the tile list; the gathered operand must equal the
    concatenation bit for bit and the product must match fp32."""
    torch.manual_seed(M + N + helpers)
    shards = [(torch.randn(M // world, K, device=DEV) * 0.5).to(BF) for _ in range(world)]
    B = (torch.randn(N, K, device=DEV) * 0.1).to(BF)
    bias = torch.randn(N, device=DEV).to(BF)
    ptrs = [t.data_ptr() for t in shards]
    X = torch.cat(shards, 0)
    ref = X.float() @ B.float().t() + bias.float()
    for rank in (0, world - 1):
        out, Xg = C.gemm_ag(ptrs, rank, M // world, K, B, False, 1, bias, False, helpers)
        assert torch.equal(Xg, X)
        assert (out.float() - ref).abs().max().item() < 0.05 * ref.abs().max().item() + 0.05
    _status_ok()


@pytest.mark.parametrize("dtype", [BF, torch.float32])
def test_vocab_parallel_embedding_push_and_pull(dtype):
    """The push / pull kernels of the row-split embedding table, with four local buffers standing in for the four
    ranks' token shards: every row arrives exactly once (stale rows are NaN, so a row nobody wrote cannot pass), ids
    outside the vocabulary give zero rows, and the pulled gradient equals the dense scatter-add."""
    torch.manual_seed(8)
    world, Ms, Cd, Vl = 4, 96, 256, 50
    M, V = world * Ms, world * Vl
    table = torch.randn(V, Cd, device=DEV).to(dtype)
    idx = torch.randint(0, V, (M,), device=DEV)
    idx[5], idx[M - 1] = V + 3, -1                                  # strays
    shards = [torch.full((Ms, Cd), float("nan"), device=DEV, dtype=dtype) for _ in range(world)]
    ptrs = [t.data_ptr() for t in shards]
    for r in range(world):
        C.embedding_vp_push(idx, table[r * Vl:(r + 1) * Vl].contiguous(), ptrs, Ms, r * Vl, V, r == 0)
    got = torch.cat(shards, 0)
    ok = (idx >= 0) & (idx < V)
    ref = torch.where(ok.unsqueeze(1), table[idx.clamp(0, V - 1)], torch.zeros((), device=DEV, dtype=dtype))
    assert torch.equal(got, ref)
    dx = [torch.randn(Ms, Cd, device=DEV).to(dtype) for _ in range(world)]
    dref = torch.zeros(V, Cd, device=DEV)
    dref.index_add_(0, idx[ok], torch.cat(dx, 0).float()[ok])
    for r in range(world):
        dw = torch.zeros(Vl, Cd, device=DEV)
        C.embedding_vp_pull_bwd(idx, [t.data_ptr() for t in dx], dw, Ms, r * Vl, dx[0])
        assert (dw - dref[r * Vl:(r + 1) * Vl]).abs().max().item() < 1e-4
    _status_ok()


@pytest.mark.parametrize("rms", [False, True])
def test_norm_fork_writes_into_a_caller_buffer(rms):
    """`fork(x, out=buf)`: the normalised rows land in `buf` (the input slot of a collective in the tensor-parallel
    blocks), values and gradients equal those of the call that allocates its own output, and `buf` itself gains no
    autograd history."""
    torch.manual_seed(4)
    M, Cd = 384, 768
    x = torch.randn(M, Cd, device=DEV).to(BF)
    w = (1 + 0.1 * torch.randn(Cd, device=DEV)).to(BF)
    b = (0.1 * torch.randn(Cd, device=DEV)).to(BF)
    dy = torch.randn(M, Cd, device=DEV).to(BF)
    res = []
    buf = torch.full((M, Cd), float("nan"), device=DEV, dtype=BF)
    for out in (None, buf):
        xr = x.clone().requires_grad_(True)
        wr = w.clone().requires_grad_(True)
        if rms:
            y, alias = ops.rmsnorm_fork(xr, wr, 1e-5, out=out)
        else:
            y, alias = ops.layernorm_fork(xr, wr, b, 1e-5, out=out)
        (y.float() * dy.float()).sum().add(alias.float().sum()).backward()
        res.append((y.detach().clone(), xr.grad.clone(), wr.grad.clone()))
        if out is not None:
            assert y.data_ptr() == buf.data_ptr()
    assert buf.grad_fn is None and not buf.requires_grad
    assert torch.equal(buf, res[0][0])
    for a, c in zip(res[0], res[1]):
        assert torch.equal(a, c)
    _status_ok()


@pytest.mark.parametrize("B,T,Hq,Hkv,hd", [(2, 128, 2, 2, 64), (2, 200, 3, 3, 64), (1, 384, 4, 2, 128), (1, 1024, 2, 2, 64),
                                           (1, 130, 8, 2, 64), (1, 4096, 8, 2, 128), (1, 4096, 4, 4, 64), (2, 2048, 4, 1, 64)])
def test_attention_pipelines_forward_and_backward(B, T, Hq, Hkv, hd):
    """Ragged last block, grouped-query heads, hd 128 (dQ shares the score columns in the backward kernel), and long
    sequences (32 key blocks per query tile: the in-place rescale of the forward accumulator and many iterations of
    the backward pipeline) against fp32 attention; two runs must agree to the bit in O, dK and dV (only dQ goes
    through floating-point atomics)."""
    torch.manual_seed(13)
    W = (Hq + 2 * Hkv) * hd
    qkv = (torch.randn(B, T, W, device=DEV) * 0.7).to(BF)
    do = torch.randn(B, T, Hq, hd, device=DEV).to(BF)
    qr = qkv.float().clone().requires_grad_(True)
    q = qr[..., :Hq * hd].reshape(B, T, Hq, hd)
    k = qr[..., Hq * hd:(Hq + Hkv) * hd].reshape(B, T, Hkv, hd)
    v = qr[..., (Hq + Hkv) * hd:].reshape(B, T, Hkv, hd)
    ref = ops.attention_ref(q, k, v)
    ref.backward(do.float())
    outs, grads = [], []
    for _ in range(2):
        qg = qkv.detach().requires_grad_(True)
        y = ops.causal_attention_qkv(qg, Hq, Hkv)
        y.backward(do)
        torch.cuda.synchronize()
        outs.append(y.detach().float())
        grads.append(qg.grad.float())
    _status_ok()
    assert (outs[0] - ref.detach()).abs().max().item() <= 2e-2
    assert torch.equal(outs[0], outs[1])
    scale = qr.grad.abs().max().item()
    for g in grads:
        assert (g - qr.grad).abs().max().item() <= 3e-2 * scale + 2e-2
    kv = slice(Hq * hd, W)
    assert torch.equal(grads[0][..., kv], grads[1][..., kv])


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("rows,cols", [(8192, 768), (8192, 3072), (1000, 2304), (37, 264), (5, 8), (4099, 1000)])
def test_column_sums_in_fixed_order(dtype, rows, cols):
    """Bias-gradient column sums: widths that fill strips of 3 vectors per lane exactly, ragged widths, fewer rows
    than warps; same bits on every run (warps and partial rows are folded in a fixed order)."""
    torch.manual_seed(17)
    x = torch.randn(rows, cols, device=DEV).to(dtype)
    ref = x.double().sum(0)
    runs = [C.colsum(x, None, False) for _ in range(3)]
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[1], runs[2])
    tol = 2e-3 * rows ** 0.5
    assert torch.allclose(runs[0].double(), ref, atol=tol)
    acc = torch.ones(cols, device=DEV)
    C.colsum(x, acc, True)
    assert torch.allclose(acc.double(), 1.0 + ref, atol=tol)
    _status_ok()


@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 1)])
def test_gemm_tile192_layouts_and_epilogue(a_mn, b_mn):
    torch.manual_seed(11)
    M, N, K = 520, 776, 328          # ragged in every dimension: 4 full 192-wide tiles + one of 8 columns
    A = (torch.randn(M, K, device=DEV) * 0.5).to(BF)
    W = (torch.randn(N, K, device=DEV) * 0.1).to(BF)
    b = (torch.randn(N, device=DEV) * 0.1).to(BF)
    R = torch.randn(M, N, device=DEV).to(BF)
    ref = A.float() @ W.float().t()
    a = A.t().contiguous() if a_mn else A
    w = W.t().contiguous() if b_mn else W
    y = C.gemm(a, w, bool(a_mn), bool(b_mn), tile_n=192, out_fp32=True)[0]
    assert torch.allclose(y, ref, rtol=1e-4, atol=2e-2)
    y = C.gemm(a, w, bool(a_mn), bool(b_mn), tile_n=192, epilogue=ops.EPI_BIAS_RESIDUAL, bias=b, aux_in=R)[0]
    assert torch.allclose(y.float(), ref + b.float() + R.float(), atol=5e-2, rtol=2e-2)
    act, pre = C.gemm(a, w, bool(a_mn), bool(b_mn), tile_n=192, epilogue=ops.EPI_BIAS_GELU, bias=b, want_aux_out=True)
    assert torch.allclose(pre.float(), ref + b.float(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(act.float(), ops.gelu_ref(pre.float()), atol=2e-2, rtol=2e-2)
    _status_ok()


@pytest.mark.parametrize("splits", [1, 3])
def test_gemm_tile192_accumulate_and_splitk(splits):
    torch.manual_seed(1)
    M, N, K = 384, 640, 1536
    A = (torch.randn(M, K, device=DEV) * 0.5).to(BF)
    B = (torch.randn(N, K, device=DEV) * 0.5).to(BF)
    ref = A.float() @ B.float().t()
    acc = torch.full((M, N), 2.0, device=DEV)
    C.gemm(A, B, out=acc, accumulate=True, tile_n=192, splits=splits)
    _status_ok()
    assert torch.allclose(acc, ref + 2.0, rtol=1e-4, atol=5e-2)


def test_clip_grad_norm_kernels():
    """sumsq -> coefficient -> in-place scaling, all on the device, against torch.nn.utils.clip_grad_norm_."""
    torch.manual_seed(9)
    for n, scale, max_norm in ((1_000_003, 1.0, 5.0), (4096, 1e-3, 1.0), (70_000_000, 0.5, 1.0)):
        g = (torch.randn(n, device=DEV) * 0.01).contiguous()
        ref = g.clone()
        ref_norm = float(ref.double().norm()) * scale
        coef = min(1.0, max_norm / (ref_norm + 1e-6))
        out = torch.zeros(2, device=DEV)
        C.clip_grad_norm_(g, max_norm, scale, out)
        assert abs(float(out[0]) - ref_norm) < 1e-4 * max(1.0, ref_norm)
        assert abs(float(out[1]) - coef) < 1e-5
        assert torch.allclose(g, ref * coef, rtol=1e-5, atol=1e-9)
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_deterministic_embedding_gradient(dtype):
    """Sorted segment reduction of the token-embedding gradient: equals index_add in float64, is bit-identical across
    runs, handles heavy repetition, a vocabulary shard, and leaves the position gradient to the regular kernel."""
    torch.manual_seed(12)
    B, T, Cdim, V = 4, 256, 96, 500
    idx = torch.randint(0, V, (B, T), device=DEV)
    idx[0, :200] = 7                                           # one token repeated 200 times
    dout = torch.randn(B, T, Cdim, device=DEV).to(dtype)
    ref = torch.zeros(V, Cdim, device=DEV, dtype=torch.float64)
    ref.index_add_(0, idx.reshape(-1), dout.reshape(-1, Cdim).double())
    runs = []
    for _ in range(3):
        dw = torch.zeros(V, Cdim, device=DEV)
        dp = torch.zeros(T, Cdim, device=DEV)
        C.embedding_bwd(idx, dout, dw, dp, 0, V, True)
        runs.append(dw.clone())
        assert torch.allclose(dp.double(), dout.double().sum(0), atol=1e-3)
    assert torch.equal(runs[0], runs[1]) and torch.equal(runs[1], runs[2])
    assert torch.allclose(runs[0].double(), ref, atol=1e-2 if dtype == BF else 1e-4, rtol=1e-3)
    # accumulation into an existing buffer, and a vocabulary shard [100, 300)
    dw = torch.ones(200, Cdim, device=DEV)
    C.embedding_bwd(idx, dout, dw, None, 100, 300, True)
    assert torch.allclose(dw.double(), 1.0 + ref[100:300], atol=1e-2 if dtype == BF else 1e-4, rtol=1e-3)
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("world", [2, 8])
def test_symmetric_collective_kernels_on_one_gpu(dtype, world):
    """The peer-pointer branch of the all-reduce / all-gather kernels with `world` local buffers standing in for the
    ranks' copies.  The kernels wait for nothing, so the ranks' launches simply run one after the other."""
    torch.manual_seed(23)
    n = 4096 * world + (16 * world // (4 if dtype == torch.float32 else 2)) * 3
    esize = 4 if dtype == torch.float32 else 2
    bufs = [torch.randn(n, device=DEV).to(dtype) for _ in range(world)]
    ptrs = [b.data_ptr() for b in bufs]
    ref = sum(b.float() for b in bufs) * 0.5
    for r in range(world):
        C.symm_allreduce(ptrs, 0, 0, n * esize, 1 if dtype == BF else 0, r, 0.5)
    torch.cuda.synchronize()
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    for b in bufs:
        assert torch.equal(b, bufs[0])
        assert (b.float() - ref).abs().max().item() <= tol * max(1.0, ref.abs().max().item())
    # all-gather of a sub-range that starts 48 bytes into the buffers
    off, per = 48 // esize, 512
    bufs = [torch.full((n,), float(r + 1), device=DEV).to(dtype) for r in range(world)]
    ptrs = [b.data_ptr() for b in bufs]
    for r in range(world):
        C.symm_allgather(ptrs, 0, off * esize, per * world * esize, r)
    torch.cuda.synchronize()
    want = torch.cat([torch.full((per,), float(r + 1), device=DEV) for r in range(world)]).to(dtype)
    for r, b in enumerate(bufs):
        assert torch.equal(b[off:off + per * world], want)
        assert torch.all(b[:off] == r + 1) and torch.all(b[off + per * world:] == r + 1)
    _status_ok()


def test_point_to_point_flag_signal_then_wait_and_bounded_timeout():
    """Signal first, then wait: the two kernels run one after the other on one stream, nothing waits for a kernel
    that has not been launched.  Then a wait for a value that nobody publishes runs out after 0.25 s, leaves the
    peer-timeout code in the status word and the context usable."""
    import time
    assert C.status_read(True) == 0
    word = torch.zeros(4, dtype=torch.int32, device=DEV)
    C.symm_signal(word.data_ptr() + 4, 7)
    C.symm_wait(word.data_ptr() + 4, 7, 1.0)
    C.symm_wait(word.data_ptr() + 4, 5, 1.0)             # already passed
    torch.cuda.synchronize()
    assert word.tolist() == [0, 7, 0, 0] and C.status_read(True) == 0
    t0 = time.time()
    C.symm_wait(word.data_ptr() + 8, 1, 0.25)            # nothing sets word[2]
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert C.status_read(True) == 2                      # peer timeout, cleared by the read
    x = torch.randn(256, 256, device=DEV).to(BF)
    assert torch.isfinite(C.gemm(x, x)[0].float()).all() and C.status_read(True) == 0


@pytest.mark.parametrize("world,npr,M,K,bias", [(2, 128, 300, 264, False), (4, 256, 1024, 768, True), (8, 128, 520, 64, True),
                                              (1, 384, 128, 128, False)])
def test_parameter_gather_gemm_on_one_gpu(world, npr, M, K, bias):
    """Collective mode 3 with `world` local buffers standing in for the ranks' copies of the weight: every launch
    plays one rank, owns `npr` rows and has NaN everywhere else, so an output without NaN proves that every
    chunk was fetched from its owner before the GEMM read it (helper and GEMM CTAs are in the same launch)."""
    torch.manual_seed(29)
    N = npr * world
    Wt = (torch.randn(N, K, device=DEV) * 0.2).to(BF)
    x = torch.randn(M, K, device=DEV).to(BF)
    b = torch.randn(N, device=DEV).to(BF) if bias else None
    ref = x.float() @ Wt.float().t() + (b.float() if bias else 0.0)
    copies = []
    for r in range(world):
        c = torch.full((N, K), float("nan"), device=DEV, dtype=BF)
        c[r * npr:(r + 1) * npr] = Wt[r * npr:(r + 1) * npr]
        copies.append(c)
    ptrs = [copies[r].data_ptr() + r * npr * K * 2 for r in range(world)]
    for r in range(world):
        y = C.gemm_param_gather(x, copies[r], ptrs, r, epilogue=ops.EPI_BIAS if bias else ops.EPI_NONE, bias=b)[0]
        torch.cuda.synchronize()
        assert torch.isfinite(y.float()).all(), f"rank {r}: a chunk was read before it arrived"
        assert torch.allclose(y.float(), ref, atol=6e-2, rtol=2e-2)
        assert torch.equal(copies[r], Wt)                  # the local copy is complete afterwards
        # later ranks must still find NaN-free *owned* rows in the earlier ranks' copies: restore the stale state
        if r + 1 < world:
            keep = copies[r][r * npr:(r + 1) * npr].clone()
            copies[r].fill_(float("nan"))
            copies[r][r * npr:(r + 1) * npr] = keep
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("V,vocab,shards", [(512, 500, 2), (1024, 1000, 4), (96, 50, 3)])
def test_vocab_parallel_xent_kernels_match_full_softmax(dtype, V, vocab, shards):
    """The slices of one [M, V] logits tensor are processed as the ranks of a group would process them (same
    kernels, one table in local memory); loss rows and gradient must equal cross entropy over the full row."""
    torch.manual_seed(6)
    M, Vl = 37, V // shards
    full = (torch.randn(M, V, device=DEV) * 3).to(dtype)
    tgt = torch.randint(0, vocab, (M,), device=DEV)
    ref_in = full.float()[:, :vocab].clone().requires_grad_(True)
    ref_rows = torch.nn.functional.cross_entropy(ref_in, tgt, reduction="none")
    ref_rows.mean().backward()
    table = torch.zeros(shards, M, 3, device=DEV)
    slices = [full[:, r * Vl:(r + 1) * Vl].contiguous() for r in range(shards)]
    for r, sl in enumerate(slices):
        C.xent_vp_stats(sl, tgt, [table.data_ptr()], r, r * Vl, vocab)
    for r, sl in enumerate(slices):
        rows = C.xent_vp_grad(sl, tgt, table, r * Vl, vocab, 1.0 / M)
        tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        assert torch.allclose(rows, ref_rows, **tol)
    grad = torch.cat(slices, 1).float()
    assert torch.all(grad[:, vocab:] == 0)
    gtol = dict(atol=1e-6, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-3, rtol=3e-2)
    assert torch.allclose(grad[:, :vocab], ref_in.grad, **gtol)
    _status_ok()


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("name", ["sum", "mean", "max", "min"])
@pytest.mark.parametrize("shape,dim", [((7, 33, 5), 1), ((6, 40), -1), ((3, 4, 5, 6), 0), ((257,), 0)])
def test_reduce_forward_backward(name, dtype, shape, dim):
    torch.manual_seed(3)
    x = torch.randn(*shape, device=DEV).to(dtype)
    xr = x.float().clone().requires_grad_(True)
    xg = x.clone().requires_grad_(True)
    for keepdim in (False, True):
        y = ops.reduce(name, xg, dim, keepdim)
        ref = getattr(torch, name)(xr, dim=dim, keepdim=keepdim)
        ref = ref if name in ("sum", "mean") else ref.values
        tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=6e-2, rtol=2e-2)
        assert y.shape == ref.shape and y.dtype == dtype
        assert torch.allclose(y.float(), ref, **tol)
    g = torch.randn_like(ref)
    (gx,) = torch.autograd.grad(y, xg, g.to(dtype))
    (gr,) = torch.autograd.grad(ref, xr, g)
    assert torch.allclose(gx.float(), gr, atol=2e-2 if dtype == BF else 1e-6, rtol=2e-2 if dtype == BF else 1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_slice_split_stack_repeat(dtype):
    torch.manual_seed(4)
    x = torch.randn(4, 9, 10, device=DEV).to(dtype).requires_grad_(True)
    xr = x.detach().clone().requires_grad_(True)
    y = ops.slice_nd(x, [1, 0, 2], [4, 9, 10], [1, 2, 3])
    ref = xr[1:4, 0:9:2, 2:10:3]
    assert torch.equal(y, ref.contiguous())
    g = torch.randn_like(y)
    assert torch.equal(torch.autograd.grad(y, x, g)[0], torch.autograd.grad(ref, xr, g)[0])

    parts, rparts = ops.split(x, 4, 1), torch.split(xr, 4, 1)
    assert len(parts) == len(rparts) == 3
    for a, b in zip(parts, rparts):
        assert torch.equal(a, b.contiguous())
    gs = [torch.randn_like(a) for a in parts]
    ga = torch.autograd.grad(parts, x, gs)[0]
    gb = torch.autograd.grad(rparts, xr, gs)[0]
    assert torch.equal(ga, gb)

    for dim in (0, 1, 3, -1):
        s, sr = ops.stack([x, x * 2], dim), torch.stack([xr, xr * 2], dim)
        assert torch.equal(s, sr)
        g = torch.randn_like(s)
        assert torch.allclose(torch.autograd.grad(s, x, g)[0].float(), torch.autograd.grad(sr, xr, g)[0].float(),
                              atol=2e-2, rtol=2e-2)

    for dim in (0, 1, 2):
        r, rr = ops.repeat_interleave(x, 3, dim), torch.repeat_interleave(xr, 3, dim=dim)
        assert torch.equal(r, rr)
        g = torch.randn_like(r)
        assert torch.allclose(torch.autograd.grad(r, x, g)[0].float(), torch.autograd.grad(rr, xr, g)[0].float(),
                              atol=5e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_masked_fill_and_outer(dtype):
    torch.manual_seed(5)
    x = torch.randn(3, 8, 8, device=DEV).to(dtype).requires_grad_(True)
    xr = x.detach().clone().requires_grad_(True)
    for mask in (torch.triu(torch.ones(8, 8, device=DEV), 1).bool(), torch.triu(torch.ones(8, 8, device=DEV), 1).to(dtype)):
        y = ops.masked_fill(x, mask, -1e4)
        ref = xr.masked_fill(mask != 0, -1e4)
        assert torch.equal(y, ref)
        g = torch.randn_like(y)
        assert torch.equal(torch.autograd.grad(y, x, g)[0], torch.autograd.grad(ref, xr, g)[0])
    a = torch.randn(37, device=DEV).to(dtype).requires_grad_(True)
    b = torch.randn(70, device=DEV).to(dtype).requires_grad_(True)
    ar, br = a.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    o, orf = ops.outer(a, b), torch.outer(ar, br)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=8e-2, rtol=2e-2)
    assert torch.allclose(o.float(), orf, **tol)
    g = torch.randn_like(orf)
    da, db = torch.autograd.grad(o, (a, b), g.to(dtype))
    dar, dbr = torch.autograd.grad(orf, (ar, br), g)
    assert torch.allclose(da.float(), dar, **tol) and torch.allclose(db.float(), dbr, **tol)
    _status_ok()

