"""The allocation-free LayerNorm backward, called through its exported C symbol.

Some users of the kernel library cannot hand it scratch memory: code running inside a CUDA
graph capture, a serving loop that must not touch the allocator, a plug-in whose host owns all
device memory.  ``titb_layernorm_bwd_noalloc`` serves them from an array built into the library.
This test loads ``libtitb200_kernels.so`` with ctypes -- no Python binding in between -- runs the
entry point twice in a row on different data and checks both results against the regular entry
point (``titb_layernorm_bwd``, which takes caller-provided scratch), plus the size limit.
It sits last in collection order so that a failure here cannot hide any other test's result.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "tinyinfinitrain_b200",
                   "libtitb200_kernels.so")
MAX_C = 2048


def _lib():
    lib = ctypes.CDLL(LIB)
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    lib.titb_layernorm_bwd_noalloc.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ll, ci, ci, ci, vp]
    lib.titb_layernorm_bwd_noalloc.restype = ci
    lib.titb_layernorm_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, ll, ci, ci, ci, vp, vp]   # ..., dres, stream
    lib.titb_layernorm_bwd.restype = ci
    lib.titb_layernorm_bwd_blocks.argtypes = [ll]
    lib.titb_layernorm_bwd_blocks.restype = ci
    lib.titb_strerror.argtypes = [ci]
    lib.titb_strerror.restype = ctypes.c_char_p
    return lib


def _case(seed, rows, C, dtype):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, C, device="cuda", generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(C, device="cuda", generator=g)).to(dtype)
    dy = torch.randn(rows, C, device="cuda", generator=g).to(dtype)
    xf = x.float()
    mean = xf.mean(-1)
    rstd = torch.rsqrt(xf.var(-1, unbiased=False) + 1e-5)
    return x, w, dy, mean.contiguous(), rstd.contiguous()


@pytest.mark.parametrize("dtype,code", [(torch.bfloat16, 1), (torch.float32, 0)])
def test_noalloc_layernorm_bwd_matches_regular_entry_point(dtype, code):
    lib = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (rows, C) in enumerate([(1000, 768), (333, 1600)]):  # two calls in a row share the scratch
        x, w, dy, mean, rstd = _case(100 + call, rows, C, dtype)
        dx_a, dx_b = torch.empty_like(x), torch.empty_like(x)
        dw_a, db_a = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
        dw_b, db_b = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
        scratch = torch.empty(2 * lib.titb_layernorm_bwd_blocks(rows) * C, device="cuda")
        p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        rc = lib.titb_layernorm_bwd_noalloc(p(dy), p(x), p(w), p(mean), p(rstd), p(dx_a), p(dw_a), p(db_a), rows, C,
                                            code, 0, stream)
        assert rc == 0, lib.titb_strerror(rc)
        rc = lib.titb_layernorm_bwd(p(dy), p(x), p(w), p(mean), p(rstd), p(dx_b), p(dw_b), p(db_b), p(scratch), rows,
                                    C, code, 0, None, stream)
        assert rc == 0, lib.titb_strerror(rc)
        torch.cuda.synchronize()
        tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=6e-2, rtol=3e-2)
        assert torch.allclose(dx_a.float(), dx_b.float(), **tol)
        assert torch.allclose(dw_a, dw_b, atol=1e-3, rtol=1e-3)
        assert torch.allclose(db_a, db_b, atol=1e-3, rtol=1e-3)
        # and against plain PyTorch fp32 math
        xr, wr = x.float().clone().requires_grad_(True), w.float().clone().requires_grad_(True)
        br = torch.zeros(C, device="cuda", requires_grad=True)
        torch.nn.functional.layer_norm(xr, (C,), wr, br, 1e-5).backward(dy.float())
        wtol = dict(atol=1e-3, rtol=1e-3) if dtype == torch.float32 else dict(atol=0.5, rtol=5e-2)
        assert torch.allclose(dx_a.float(), xr.grad, **tol)
        assert torch.allclose(dw_a, wr.grad, **wtol)
        assert torch.allclose(db_a, br.grad, **wtol)


def test_noalloc_rejects_rows_wider_than_its_scratch():
    lib = _lib()
    C = MAX_C + 8
    x, w, dy, mean, rstd = _case(7, 4, C, torch.float32)
    dx, dw, db = torch.empty_like(x), torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    rc = lib.titb_layernorm_bwd_noalloc(p(dy), p(x), p(w), p(mean), p(rstd), p(dx), p(dw), p(db), 4, C, 0, 0,
                                        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    assert b"TITB_NOALLOC_LAYERNORM_MAX_C" in lib.titb_strerror(rc)
