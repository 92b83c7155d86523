"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

import tinyinfinitrain_b200 as tit
from tinyinfinitrain_b200 import ops
from tinyinfinitrain_b200._lib import C

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16


def _status_ok():
    torch.cuda.synchronize()
    assert C.status_read(True) == 0


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [
    (128, 128, 64, 0, 0), (256, 512, 512, 0, 0), (1000, 776, 520, 0, 0), (512, 768, 2048, 0, 1),
    (768, 1024, 1024, 1, 1), (8, 8, 8, 0, 0), (136, 72, 40, 1, 0), (2048, 50304, 128, 0, 0),
])
def test_gemm_tcgen05(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    A = (torch.randn(M, K, device=DEV) * 0.5).to(BF)
    B = (torch.randn(N, K, device=DEV) * 0.5).to(BF)
    ref = A.float() @ B.float().t()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = C.gemm(a, b, bool(a_mn), bool(b_mn), out_fp32=True)[0]
    _status_ok()
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-3 * math.sqrt(K))
    out16 = C.gemm(a, b, bool(a_mn), bool(b_mn))[0]
    assert torch.allclose(out16.float(), ref, rtol=2e-2, atol=2e-2 * math.sqrt(K))


@pytest.mark.parametrize("tile_n", [128, 256])
@pytest.mark.parametrize("splits", [1, 3])
def test_gemm_tiles_and_splitk(tile_n, splits):
    torch.manual_seed(1)
    M, N, K = 384, 640, 1536
    A = (torch.randn(M, K, device=DEV) * 0.5).to(BF)
    B = (torch.randn(N, K, device=DEV) * 0.5).to(BF)
    ref = A.float() @ B.float().t()
    acc = torch.full((M, N), 2.0, device=DEV)
    C.gemm(A, B, out=acc, accumulate=True, tile_n=tile_n, splits=splits)
    _status_ok()
    assert torch.allclose(acc, ref + 2.0, rtol=1e-4, atol=5e-2)


@pytest.mark.parametrize("tile_n", [128, 192, 256])
@pytest.mark.parametrize("splits,accumulate", [(1, False), (1, True), (4, False), (4, True), (0, False)])
def test_gemm_weight_gradient_form_fp32_out(tile_n, splits, accumulate):
    """dW = dY^T X (both operands MN-major, long reduction, fp32 result): stored, accumulated, and split over K with the
    partial tiles added in the output (zero-filled first when it does not accumulate); splits = 0 lets the planner
    choose.  Ragged in both output dimensions."""
    torch.manual_seed(6)
    tokens, n_out, k_in = 4096, 328, 776
    dY = (torch.randn(tokens, n_out, device=DEV) * 0.5).to(BF)
    X = (torch.randn(tokens, k_in, device=DEV) * 0.5).to(BF)
    ref = dY.float().t() @ X.float()
    out = torch.full((n_out, k_in), 3.0, device=DEV)
    C.gemm(dY, X, True, True, out=out, accumulate=accumulate, tile_n=tile_n, splits=splits)
    _status_ok()
    want = ref + 3.0 if accumulate else ref
    assert torch.allclose(out, want, rtol=1e-4, atol=5e-2)
    al = torch.tensor([0.5], device=DEV)
    out.fill_(1.0)
    C.gemm(dY, X, True, True, out=out, accumulate=True, tile_n=tile_n, splits=splits, alpha=al)
    assert torch.allclose(out, 0.5 * ref + 1.0, rtol=1e-4, atol=5e-2)
    _status_ok()


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [
    (256, 256, 64, 0, 0), (512, 768, 512, 0, 0), (1000, 776, 520, 0, 0), (1024, 768, 2048, 0, 1),
    (768, 1024, 1024, 1, 1), (136, 264, 40, 1, 0), (2048, 2304, 768, 0, 0), (8192, 768, 768, 0, 1),
])
def test_gemm_cta_pairs(M, N, K, a_mn, b_mn):
    """tile_n = 512: two CTAs of a cluster share each 256 x 256 tile (tcgen05 cta_group::2), each staging its own
    half of the operands.  Row counts that leave the second CTA of the last pair partly or wholly outside the matrix,
    ragged widths, all operand layouts, many tiles per pair (both accumulator buffers and every ring stage reused)."""
    torch.manual_seed(8)
    A = (torch.randn(M, K, device=DEV) * 0.5).to(BF)
    B = (torch.randn(N, K, device=DEV) * 0.5).to(BF)
    ref = A.float() @ B.float().t()
    a = A.t().contiguous() if a_mn else A
    b = B.t().contiguous() if b_mn else B
    out = C.gemm(a, b, bool(a_mn), bool(b_mn), out_fp32=True, tile_n=512)[0]
    _status_ok()
    assert torch.allclose(out, ref, rtol=1e-4, atol=1e-3 * math.sqrt(K))
    out16 = C.gemm(a, b, bool(a_mn), bool(b_mn), tile_n=512)[0]
    _status_ok()
    assert torch.allclose(out16.float(), ref, rtol=2e-2, atol=2e-2 * math.sqrt(K))


def test_gemm_cta_pairs_epilogues_and_splits():
    torch.manual_seed(9)
    M, N, K = 1160, 776, 328
    A = (torch.randn(M, K, device=DEV) * 0.5).to(BF)
    W = (torch.randn(N, K, device=DEV) * 0.1).to(BF)
    b = (torch.randn(N, device=DEV) * 0.1).to(BF)
    R = torch.randn(M, N, device=DEV).to(BF)
    ref = A.float() @ W.float().t()
    y = C.gemm(A, W, epilogue=ops.EPI_BIAS_RESIDUAL, bias=b, aux_in=R, tile_n=512)[0]
    assert torch.allclose(y.float(), ref + b.float() + R.float(), atol=5e-2, rtol=2e-2)
    act, pre = C.gemm(A, W, epilogue=ops.EPI_BIAS_GELU, bias=b, want_aux_out=True, tile_n=512)
    assert torch.allclose(pre.float(), ref + b.float(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(act.float(), ops.gelu_ref(pre.float()), atol=2e-2, rtol=2e-2)
    y = C.gemm(A, W, epilogue=ops.EPI_DGELU, aux_in=pre, tile_n=512)[0]
    x = pre.float().requires_grad_(True)
    ops.gelu_ref(x).sum().backward()
    assert torch.allclose(y.float(), ref * x.grad, atol=5e-2, rtol=3e-2)
    # weight-gradient form, fp32 accumulate, split over K
    tokens = 4096
    dY = (torch.randn(tokens, 520, device=DEV) * 0.5).to(BF)
    X = (torch.randn(tokens, 776, device=DEV) * 0.5).to(BF)
    acc = torch.full((520, 776), 2.0, device=DEV)
    C.gemm(dY, X, True, True, out=acc, accumulate=True, tile_n=512, splits=4)
    assert torch.allclose(acc, dY.float().t() @ X.float() + 2.0, rtol=1e-4, atol=5e-2)
    _status_ok()


def test_gemm_epilogues():
    torch.manual_seed(2)
    M, N, K = 520, 776, 264
    A = (torch.randn(M, K, device=DEV) * 0.5).to(BF)
    W = (torch.randn(N, K, device=DEV) * 0.1).to(BF)
    b = (torch.randn(N, device=DEV) * 0.1).to(BF)
    R = torch.randn(M, N, device=DEV).to(BF)
    ref = A.float() @ W.float().t()
    y = C.gemm(A, W, epilogue=ops.EPI_BIAS, bias=b)[0]
    assert torch.allclose(y.float(), ref + b.float(), atol=3e-2, rtol=2e-2)
    act, pre = C.gemm(A, W, epilogue=ops.EPI_BIAS_GELU, bias=b, want_aux_out=True)
    assert torch.allclose(pre.float(), ref + b.float(), atol=3e-2, rtol=2e-2)
    assert torch.allclose(act.float(), ops.gelu_ref(pre.float()), atol=2e-2, rtol=2e-2)
    y = C.gemm(A, W, epilogue=ops.EPI_BIAS_RESIDUAL, bias=b, aux_in=R)[0]
    assert torch.allclose(y.float(), ref + b.float() + R.float(), atol=5e-2, rtol=2e-2)
    x = pre.float().requires_grad_(True)
    ops.gelu_ref(x).sum().backward()
    y = C.gemm(A, W, epilogue=ops.EPI_DGELU, aux_in=pre)[0]
    assert torch.allclose(y.float(), ref * x.grad, atol=5e-2, rtol=3e-2)
    al = torch.tensor([0.25], device=DEV)
    y = C.gemm(A, W, alpha=al, out_fp32=True)[0]
    assert torch.allclose(y, 0.25 * ref, atol=1e-2, rtol=1e-3)
    _status_ok()


def test_sgemm_fp32():
    torch.manual_seed(3)
    A, B = torch.randn(70, 33, device=DEV), torch.randn(33, 45, device=DEV)
    assert torch.allclose(C.sgemm(A, B), A @ B, atol=1e-4)
    assert torch.allclose(C.sgemm(A.t().contiguous(), B, True, False), A @ B, atol=1e-4)
    assert torch.allclose(C.sgemm(A, B.t().contiguous(), False, True), A @ B, atol=1e-4)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("rows,Cdim", [(64, 768), (1000, 1600), (33, 2048), (17, 4096), (5, 100)])
def test_layernorm(dtype, rows, Cdim):
    torch.manual_seed(4)
    x = torch.randn(rows, Cdim, device=DEV).to(dtype)
    w = (1 + 0.1 * torch.randn(Cdim, device=DEV)).to(dtype)
    b = (0.1 * torch.randn(Cdim, device=DEV)).to(dtype)
    dy = torch.randn(rows, Cdim, device=DEV).to(dtype)
    xr, wr, br = (t.float().detach().clone().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (Cdim,), wr, br, 1e-5)
    yr.backward(dy.float())
    xg, wg, bg = (t.detach().requires_grad_(True) for t in (x, w, b))
    y = ops.layernorm(xg, wg, bg, 1e-5)
    y.backward(dy)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=6e-2, rtol=3e-2)
    assert torch.allclose(y.float(), yr, **tol)
    assert torch.allclose(xg.grad.float(), xr.grad, **tol)
    wtol = dict(atol=1e-3, rtol=1e-3) if dtype == torch.float32 else dict(atol=0.5, rtol=5e-2)
    assert torch.allclose(wg.grad.float(), wr.grad, **wtol)
    assert torch.allclose(bg.grad.float(), br.grad, **wtol)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("rows,Cdim", [(64, 2048), (100, 4096), (7, 72)])
def test_rmsnorm(dtype, rows, Cdim):
    torch.manual_seed(5)
    x = torch.randn(rows, Cdim, device=DEV).to(dtype)
    w = (1 + 0.1 * torch.randn(Cdim, device=DEV)).to(dtype)
    dy = torch.randn(rows, Cdim, device=DEV).to(dtype)
    xr, wr = x.float().detach().clone().requires_grad_(True), w.float().detach().clone().requires_grad_(True)
    yr = ops.rmsnorm_ref(xr, wr, 1e-5)
    yr.backward(dy.float())
    xg, wg = x.detach().requires_grad_(True), w.detach().requires_grad_(True)
    y = ops.rmsnorm(xg, wg, 1e-5)
    y.backward(dy)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=6e-2, rtol=3e-2)
    assert torch.allclose(y.float(), yr, **tol)
    assert torch.allclose(xg.grad.float(), xr.grad, **tol)
    wtol = dict(atol=1e-3, rtol=1e-3) if dtype == torch.float32 else dict(atol=0.5, rtol=5e-2)
    assert torch.allclose(wg.grad.float(), wr.grad, **wtol)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_gelu_swiglu_rope(dtype):
    torch.manual_seed(6)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    x = torch.randn(37, 264, device=DEV).to(dtype)
    dy = torch.randn(37, 264, device=DEV).to(dtype)
    xr = x.float().clone().requires_grad_(True); ops.gelu_ref(xr).backward(dy.float())
    xg = x.detach().requires_grad_(True); y = ops.gelu(xg); y.backward(dy)
    assert torch.allclose(y.float(), ops.gelu_ref(x.float()), **tol)
    assert torch.allclose(xg.grad.float(), xr.grad, **tol)
    x = torch.randn(19, 2 * 256, device=DEV).to(dtype)
    dy = torch.randn(19, 256, device=DEV).to(dtype)
    xr = x.float().clone().requires_grad_(True)
    g, u = xr.chunk(2, -1); (torch.nn.functional.silu(g) * u).backward(dy.float())
    xg = x.detach().requires_grad_(True); y = ops.swiglu(xg); y.backward(dy)
    g0, u0 = x.float().chunk(2, -1)
    assert torch.allclose(y.float(), torch.nn.functional.silu(g0) * u0, **tol)
    assert torch.allclose(xg.grad.float(), xr.grad, **tol)
    x = torch.randn(2, 33, 4, 64, device=DEV).to(dtype)
    dy = torch.randn_like(x)
    xr = x.float().clone().requires_grad_(True); ops.rope_ref(xr, 3, 500000.0).backward(dy.float())
    xg = x.detach().requires_grad_(True); y = ops.rope(xg, 3, 500000.0); y.backward(dy)
    assert torch.allclose(y.float(), ops.rope_ref(x.float(), 3, 500000.0), **tol)
    assert torch.allclose(xg.grad.float(), xr.grad, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_embedding(dtype):
    torch.manual_seed(7)
    V, T, Cdim, B = 300, 24, 64, 3
    wte = torch.randn(V, Cdim, device=DEV).to(dtype)
    wpe = torch.randn(T, Cdim, device=DEV).to(dtype)
    idx = torch.randint(0, V, (B, T), device=DEV)
    dy = torch.randn(B, T, Cdim, device=DEV).to(dtype)
    a, p = wte.detach().requires_grad_(True), wpe.detach().requires_grad_(True)
    y = ops.embedding(idx, a, p)
    y.backward(dy)
    ar, pr = wte.float().clone().requires_grad_(True), wpe.float().clone().requires_grad_(True)
    yr = torch.nn.functional.embedding(idx, ar) + pr[None]
    yr.backward(dy.float())
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=5e-2, rtol=2e-2)
    assert torch.allclose(y.float(), yr, **tol)
    assert torch.allclose(a.grad.float(), ar.grad, **tol)
    assert torch.allclose(p.grad.float(), pr.grad, **tol)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
@pytest.mark.parametrize("rows,V,ld", [(64, 50257, 50304), (33, 1000, 1000), (8, 77, 80)])
def test_cross_entropy(dtype, rows, V, ld):
    torch.manual_seed(8)
    logits = (torch.randn(rows, ld, device=DEV) * 2).to(dtype)
    tgt = torch.randint(0, V, (rows,), device=DEV)
    lr = logits.float()[:, :V].detach().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(lr, tgt)
    (ref * 1.5).backward()
    lg = logits.detach().requires_grad_(True)
    loss = ops.cross_entropy(lg, tgt, V)
    (loss * 1.5).backward()
    assert abs(loss.item() - ref.item()) < (1e-4 if dtype == torch.float32 else 2e-2)
    tol = dict(atol=1e-6, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-3, rtol=2e-2)
    assert torch.allclose(lg.grad.float()[:, :V], lr.grad, **tol)
    assert lg.grad[:, V:].abs().sum().item() == 0


def test_lm_head_loss_fused():
    torch.manual_seed(9)
    M, Cdim, V, Vp = 256, 128, 1000, 1024
    x = (torch.randn(M, Cdim, device=DEV)).to(BF)
    w = (torch.randn(Vp, Cdim, device=DEV) * 0.05).to(BF)
    tgt = torch.randint(0, V, (M,), device=DEV)
    xr, wr = x.float().clone().requires_grad_(True), w.float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy((xr @ wr.t())[:, :V], tgt)
    (ref * 2.0).backward()
    xg, wg = x.detach().requires_grad_(True), w.detach().requires_grad_(True)
    loss = ops.lm_head_loss(xg, wg, tgt, V)
    (loss * 2.0).backward()
    assert abs(loss.item() - ref.item()) < 2e-2
    assert torch.allclose(xg.grad.float(), xr.grad, atol=2e-3, rtol=5e-2)
    assert torch.allclose(wg.grad.float(), wr.grad, atol=2e-3, rtol=5e-2)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_softmax_any_axis(dtype):
    torch.manual_seed(10)
    x = torch.randn(3, 17, 9, device=DEV).to(dtype)
    dy = torch.randn_like(x)
    for dim in (0, 1, 2, -1):
        xr = x.float().clone().requires_grad_(True); yr = torch.softmax(xr, dim); yr.backward(dy.float())
        xg = x.detach().requires_grad_(True); y = ops.softmax(xg, dim); y.backward(dy)
        tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=1e-2, rtol=2e-2)
        assert torch.allclose(y.float(), yr, **tol)
        assert torch.allclose(xg.grad.float(), xr.grad, **tol)


def test_adam_and_sgd_flat():
    torch.manual_seed(11)
    n = 1000 + 3
    w = torch.randn(n, device=DEV); g = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV); v = torch.zeros(n, device=DEV)
    wr, mr, vr = w.clone(), m.clone(), v.clone()
    lp = torch.empty(n, device=DEV, dtype=BF)
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    for t in range(1, 4):
        C.adam_flat(w, lp, g, m, v, lr, b1, b2, eps, wd, t, 1.0)
        mr = b1 * mr + (1 - b1) * g; vr = b2 * vr + (1 - b2) * g * g
        wr = wr - lr * ((mr / (1 - b1 ** t)) / ((vr / (1 - b2 ** t)).sqrt() + eps) + wd * wr)
    assert torch.allclose(w, wr, atol=1e-5)
    assert torch.allclose(lp.float(), wr, atol=1e-2, rtol=1e-2)
    w2 = torch.randn(n, device=DEV); w2r = w2.clone()
    C.sgd_flat(w2, None, g, 0.1)
    assert torch.allclose(w2, w2r - 0.1 * g, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, BF])
def test_elementwise_family(dtype):
    torch.manual_seed(12)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    x = (torch.rand(5, 37, device=DEV) + 0.5).to(dtype)
    dy = torch.randn(5, 37, device=DEV).to(dtype)
    cases = [("neg", 0, lambda t: -t), ("reciprocal", 0, lambda t: 1 / t), ("sin", 0, torch.sin), ("cos", 0, torch.cos),
             ("tanh", 0, torch.tanh), ("pow_exp", 2.0, lambda t: t ** 2.0), ("pow_base", 2.0, lambda t: 2.0 ** t),
             ("rsqrt", 0, torch.rsqrt), ("add_scalar", 1.5, lambda t: t + 1.5), ("mul_scalar", -2.0, lambda t: t * -2.0),
             ("sigmoid", 0, torch.sigmoid)]
    for name, s, ref in cases:
        xr = x.float().clone().requires_grad_(True); yr = ref(xr); yr.backward(dy.float())
        xg = x.detach().requires_grad_(True); y = ops.unary(name, xg, s); y.backward(dy)
        assert torch.allclose(y.float(), yr, **tol), name
        assert torch.allclose(xg.grad.float(), xr.grad, **tol), name
    assert torch.equal(ops.unary("equals_scalar", x, float(x[0, 0])), (x == x[0, 0]).to(dtype))
    a = torch.randn(4, 6, 8, device=DEV).to(dtype); b = (torch.rand(6, 1, device=DEV) + 0.5).to(dtype)
    for name, ref in [("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div)]:
        ar, br = a.float().clone().requires_grad_(True), b.float().clone().requires_grad_(True)
        yr = ref(ar, br); yr.backward(torch.ones_like(yr))
        ag, bg = a.detach().requires_grad_(True), b.detach().requires_grad_(True)
        y = ops.binary(name, ag, bg); y.backward(torch.ones_like(y))
        assert torch.allclose(y.float(), yr, **tol), name
        assert torch.allclose(ag.grad.float(), ar.grad, **tol), name
        assert torch.allclose(bg.grad.float(), br.grad, atol=0.3 if dtype == BF else 1e-4, rtol=3e-2), name
    t = torch.randn(3, 50, 70, device=DEV).to(dtype)
    assert torch.equal(ops.transpose(t, 1, 2), t.transpose(1, 2).contiguous())
    m2 = torch.randn(9, 11, device=DEV).to(dtype)
    assert torch.equal(ops.tril(m2, 1), torch.tril(m2, 1)) and torch.equal(ops.triu(m2, -1), torch.triu(m2, -1))
    assert torch.allclose(ops.cast(m2, torch.float32), m2.float())
    assert torch.equal(ops.cast(m2.float(), BF), m2.float().to(BF))
    cs = C.colsum(t.reshape(-1, 70).contiguous())
    assert torch.allclose(cs, t.float().reshape(-1, 70).sum(0), atol=1e-2 if dtype == BF else 1e-4)


@pytest.mark.parametrize("B,T,Hq,Hkv,hd", [(2, 128, 2, 2, 64), (1, 256, 4, 4, 64), (2, 200, 3, 3, 64), (1, 384, 4, 2, 128),
                                           (1, 1024, 2, 2, 64), (1, 130, 8, 2, 64)])
def test_attention_fwd_bwd(B, T, Hq, Hkv, hd):
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
    qg = qkv.detach().requires_grad_(True)
    out = ops.causal_attention_qkv(qg, Hq, Hkv)
    out.backward(do)
    _status_ok()
    assert torch.allclose(out.float(), ref, atol=2e-2, rtol=2e-2)
    err = (qg.grad.float() - qr.grad).abs().max().item()
    scale = qr.grad.abs().max().item()
    assert err <= 3e-2 * scale + 2e-2, (err, scale)


def test_gpt2_tiny_matches_cpu_oracle():
    from tinyinfinitrain_b200.models import GPT2, GPT2Config

    cfg = GPT2Config(block_size=128, vocab_size=1000, n_layer=2, n_head=4, n_embd=256)
    cpu = GPT2(cfg)
    gpu = GPT2(cfg, device=DEV, dtype=BF)
    g = torch.Generator().manual_seed(42)
    idx = torch.randint(0, 1000, (4, 128), generator=g)
    tgt = torch.roll(idx, -1, 1)
    _, l_cpu = cpu(idx, tgt)
    _, l_fused = gpu(idx.to(DEV), tgt.to(DEV), return_logits=False)
    logits, l_plain = gpu(idx.to(DEV), tgt.to(DEV))
    assert abs(l_cpu.item() - l_fused.item()) < 3e-2
    assert abs(l_cpu.item() - l_plain.item()) < 3e-2
    assert logits.shape == (4, 128, 1000)
    opt = tit.optim.MixedPrecisionAdam(gpu.parameters(), lr=1e-3)
    first = last = None
    for _ in range(8):
        opt.zero_grad()
        _, loss = gpu(idx.to(DEV), tgt.to(DEV), return_logits=False)
        loss.backward()
        opt.step()
        first = first if first is not None else loss.item()
        last = loss.item()
    _status_ok()
    assert last < first - 0.5, (first, last)
