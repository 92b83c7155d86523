"""The GPU tests of the opt-in kernels, run on CPU against PyTorch restatements of the kernels' contracts.  This checks
the tests themselves -- argument order, reference math, tolerances, the accumulate / residual / shard cases -- so that
a failure on a GPU points at the kernel and not at the test."""
import importlib

import pytest
import torch


def _bytes_at(ptr, nbytes):
    """A uint8 view of `nbytes` bytes of host memory at address `ptr`, found among the live CPU tensors (the tests
    hand raw addresses to the kernels, as they do on the GPU)."""
    import gc

    for o in gc.get_objects():
        if isinstance(o, torch.Tensor) and o.device.type == "cpu" and o.numel() and o.is_contiguous():
            base, size = o.data_ptr(), o.numel() * o.element_size()
            if base <= ptr and ptr + nbytes <= base + size:
                return o.view(-1).view(torch.uint8)[ptr - base: ptr - base + nbytes]
    raise LookupError(hex(ptr))


class Restated:
    """Contracts of the entry points the tests call, in plain PyTorch (fp32 math, results in the kernels' dtypes)."""

    @staticmethod
    def status_read(clear=True):
        st = Restated._status
        if clear:
            Restated._status = 0
        return st

    @staticmethod
    def symm_allreduce(ptrs, mc_ptr, byte_off, nbytes, dtype, rank, scale=1.0, max_blocks=0):
        world, dt = len(ptrs), (torch.bfloat16 if dtype == 1 else torch.float32)
        sl = nbytes // world                                  # this rank reduces and publishes its slice only
        lo = byte_off + rank * sl
        views = [_bytes_at(p + lo, sl).view(dt) for p in ptrs]
        total = sum(v.float() for v in views) * scale
        for v in views:
            v.copy_(total.to(dt))

    @staticmethod
    def symm_allgather(ptrs, mc_ptr, byte_off, nbytes, rank, max_blocks=0):
        sl = nbytes // len(ptrs)
        lo = byte_off + rank * sl
        mine = _bytes_at(ptrs[rank] + lo, sl).clone()
        for p in ptrs:
            _bytes_at(p + lo, sl).copy_(mine)

    @staticmethod
    def symm_signal(word, value):
        _bytes_at(word, 4).view(torch.int32)[0] = value

    @staticmethod
    def symm_wait(word, value, timeout_s=2.0):
        have = int(_bytes_at(word, 4).view(torch.int32)[0])
        if have - value < 0:
            Restated._status = 2                               # nothing will ever publish it here: the wait runs out

    _status = 0

    @staticmethod
    def gemm_param_gather(x, w, peer_ptrs, rank, epilogue=0, bias=None, aux_in=None, want_aux_out=False, helper_ctas=8,
                          tile_n=0):
        world = len(peer_ptrs)
        N, K = w.shape
        npr, row_bytes = N // world, K * w.element_size()
        for r in range(world):                                 # rows are fetched from the memory of the rank that owns them
            rows = _bytes_at(peer_ptrs[r], npr * row_bytes).view(w.dtype).view(npr, K)
            if rows.data_ptr() != w[r * npr].data_ptr():
                w[r * npr:(r + 1) * npr] = rows
        y = x.float() @ w.float().t()
        if bias is not None:
            y = y + bias.float()
        return [y.to(x.dtype)]

    @staticmethod
    def gemm(a, b, *args, **kwargs):
        return [(a.float() @ b.float().t()).to(a.dtype)]

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


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("world", [2, 8])
def test_symmetric_collective_test_logic(gpu_tests, monkeypatch, dtype, world):
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    gpu_tests.test_symmetric_collective_kernels_on_one_gpu(dtype, world)


def test_flag_test_logic(gpu_tests, monkeypatch):
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    gpu_tests.test_point_to_point_flag_signal_then_wait_and_bounded_timeout()


@pytest.mark.parametrize("world,npr,M,K,bias", [(2, 128, 300, 264, False), (4, 256, 64, 96, True), (1, 384, 128, 128, False)])
def test_parameter_gather_test_logic(gpu_tests, monkeypatch, world, npr, M, K, bias):
    monkeypatch.setattr(torch.cuda, "synchronize", lambda *a, **k: None)
    gpu_tests.test_parameter_gather_gemm_on_one_gpu(world, npr, M, K, bias)
