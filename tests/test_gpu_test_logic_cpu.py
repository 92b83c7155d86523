"""The GPU tests of the opt-in kernels, run on CPU against PyTorch restatements of the kernels' contracts.  This checks
the tests themselves -- argument order, reference math, tolerances, the accumulate / residual / shard cases -- so that
a failure on a GPU points at the kernel and not at the test."""
import importlib

import pytest
import torch


class Restated:
    """Contracts of the entry points the tests call, in plain PyTorch (fp32 math, results in the kernels' dtypes)."""

    @staticmethod
    def status_read(clear=True):
        return 0

    @staticmethod
    def attn_bwd_set_warps(warps):
        pass

    @staticmethod
    def colsum(x, out=None, accumulate=False, fused=False):
        s = x.float().sum(0)
        if out is None:
            return s
        out.copy_(out + s if accumulate else s)
        return out

    @staticmethod
    def layernorm_fwd(x, w, b, eps):
        xf = x.float()
        mean = xf.mean(-1)
        rstd = torch.rsqrt(xf.var(-1, unbiased=False) + eps)
        y = (xf - mean[:, None]) * rstd[:, None] * w.float() + b.float()
        return y.to(x.dtype), mean, rstd

    @staticmethod
    def rmsnorm_fwd(x, w, eps):
        xf = x.float()
        rstd = torch.rsqrt(xf.pow(2).mean(-1) + eps)
        return (xf * rstd[:, None] * w.float()).to(x.dtype), rstd

    @staticmethod
    def _norm_bwd(dy, x, w, mean, rstd, dw, db, accumulate, dres, rms):
        g, xf = dy.float(), x.float()
        n = (xf - (0 if rms else mean[:, None])) * rstd[:, None]
        dn = g * w.float()
        m1 = 0 if rms else dn.mean(-1, keepdim=True)
        dx = (dn - m1 - n * (dn * n).mean(-1, keepdim=True)) * rstd[:, None]
        if dres is not None:
            dx = dx + dres.float()
        gw, gb = (g * n).sum(0), g.sum(0)
        dw_t = dw if dw is not None else torch.zeros_like(gw)
        dw_t.copy_(dw_t + gw if (dw is not None and accumulate) else gw)
        if rms:
            return [dx.to(x.dtype), dw_t]
        db_t = db if db is not None else torch.zeros_like(gb)
        db_t.copy_(db_t + gb if (db is not None and accumulate) else gb)
        return [dx.to(x.dtype), dw_t, db_t]

    @staticmethod
    def layernorm_bwd(dy, x, w, mean, rstd, dw=None, db=None, accumulate=False, onepass=False, dres=None):
        return Restated._norm_bwd(dy, x, w, mean, rstd, dw, db, accumulate, dres, False)

    @staticmethod
    def rmsnorm_bwd(dy, x, w, rstd, dw=None, accumulate=False, onepass=False, dres=None):
        return Restated._norm_bwd(dy, x, w, None, rstd, dw, None, accumulate, dres, True)

    @staticmethod
    def xent_fused(logits, targets, V, grad_scale, write_grad, mean_scale, row_cached=False):
        lf = logits.float()[:, :V]
        lse = torch.logsumexp(lf, -1)
        loss = (lse - lf.gather(1, targets[:, None])[:, 0]).sum() * mean_scale
        if write_grad:
            p = torch.softmax(lf, -1)
            p.scatter_add_(1, targets[:, None], -torch.ones_like(p[:, :1]))
            logits[:, :V] = (p * grad_scale).to(logits.dtype)
            logits[:, V:] = 0
        return loss

    @staticmethod
    def embedding_bwd(idx, dout, dwte=None, dwpe=None, vocab_lo=0, vocab_hi=1 << 40, deterministic=False):
        flat, g = idx.reshape(-1), dout.reshape(-1, dout.shape[-1]).float()
        keep = (flat >= vocab_lo) & (flat < vocab_hi)
        dwte.index_add_(0, flat[keep] - vocab_lo, g[keep])
        if dwpe is not None:
            dwpe.add_(dout.float().sum(0))

    @staticmethod
    def clip_grad_norm_(g, max_norm, scale, out):
        norm = g.double().norm().float() * scale
        coef = torch.clamp(max_norm / (norm + 1e-6), max=1.0)
        g.mul_(coef)
        out[0], out[1] = norm, coef


@pytest.fixture
def gpu_tests(monkeypatch):
    mod = importlib.import_module("test_zzz_gpu_recent_kernels")
    monkeypatch.setattr(mod, "DEV", "cpu")
    monkeypatch.setattr(mod, "C", Restated)
    monkeypatch.setattr(mod, "_status_ok", lambda: None)
    monkeypatch.setenv("TITB_TEST_STRICT", "1")
    return mod


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1000, 1024), (37, 256), (5, 64)])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_backward_test_logic(gpu_tests, dtype, rows, cols, rms):
    gpu_tests.test_one_launch_norm_backward_matches_the_two_stage_kernels(dtype, rows, cols, rms)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1000, 2304), (37, 264), (5, 8)])
def test_column_sum_test_logic(gpu_tests, dtype, rows, cols):
    gpu_tests.test_one_launch_column_sum_matches_the_two_stage_kernel(dtype, rows, cols)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,ld,V", [(33, 1000, 1000), (16, 512, 300)])
def test_row_cached_xent_test_logic(gpu_tests, dtype, rows, ld, V):
    gpu_tests.test_row_cached_cross_entropy_matches_the_regular_kernel(dtype, rows, ld, V)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_deterministic_embedding_test_logic(gpu_tests, dtype):
    gpu_tests.test_deterministic_embedding_gradient(dtype)


def test_clip_test_logic(gpu_tests, monkeypatch):
    gpu_tests.test_clip_grad_norm_kernels()


@pytest.mark.parametrize("B,T,Hq,Hkv,hd", [(2, 128, 2, 2, 64), (1, 130, 8, 2, 64)])
def test_attention_variant_test_logic(gpu_tests, monkeypatch, B, T, Hq, Hkv, hd):
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    gpu_tests.test_attention_backward_with_two_warps_per_score_row(B, T, Hq, Hkv, hd)


def test_norm_fork_test_logic(gpu_tests, monkeypatch):
    gpu_tests.test_norm_fork_folds_the_residual_gradient(monkeypatch)
