"""The Python wrappers of the reduction / view kernels (sizes, strides, offsets, saved state of the autograd functions)
on CPU: the seven kernel entry points are replaced by PyTorch restatements of what the CUDA kernels compute, and the
GPU tests of the same wrappers are run against them."""
import importlib

import pytest
import torch

from tinyinfinitrain_b200.ops import functional as Fn


class KernelRestatement:
    """What csrc/kernels/transform.cu does, per entry point, in PyTorch."""

    @staticmethod
    def gather_view(base, sizes, strides, offset):
        return torch.as_strided(base.reshape(-1), sizes, strides, offset).clone().contiguous()

    @staticmethod
    def scatter_view_(dst, src, strides, offset, accumulate=False):
        flat, n = dst.view(-1), src.numel()
        off, t = torch.full((n,), offset), torch.arange(n)
        for d in reversed(range(src.dim())):            # the kernel peels indices innermost first
            q = t // src.shape[d]
            off += (t - q * src.shape[d]) * strides[d]
            t = q
        if accumulate:
            flat.index_add_(0, off, src.reshape(-1))
        else:
            flat[off] = src.reshape(-1)

    @staticmethod
    def reduce_dim(x, op, dim, keepdim):
        r = getattr(torch, ["sum", "mean", "max", "min"][op])(x, dim=dim, keepdim=keepdim)
        return (r, None) if op < 2 else (r.values, r.indices)

    @staticmethod
    def reduce_dim_bwd(g, idx, in_sizes, dim, scale):
        nd = len(in_sizes)
        dim %= nd
        outer = int(torch.tensor(in_sizes[:dim]).prod()) if dim else 1
        inner = int(torch.tensor(in_sizes[dim + 1:]).prod()) if dim + 1 < nd else 1
        n = in_sizes[dim]
        g2 = g.reshape(outer, 1, inner)
        if idx is None:
            return (g2 * scale).expand(outer, n, inner).reshape(in_sizes).contiguous()
        hit = torch.arange(n).view(1, n, 1) == idx.reshape(outer, 1, inner)
        return torch.where(hit, g2, torch.zeros_like(g2)).reshape(in_sizes)

    @staticmethod
    def mask_fill(x, mask, value, backward):
        m = (mask != 0).reshape(-1)
        xf = x.reshape(-1, m.numel())
        return torch.where(m, torch.zeros_like(xf) if backward else torch.full_like(xf, value), xf).reshape(x.shape)

    @staticmethod
    def outer_fwd(a, b):
        return a[:, None] * b[None, :]

    @staticmethod
    def outer_bwd(g, a, b):
        return [g @ b, g.t() @ a]


@pytest.fixture
def gpu_tests(monkeypatch):
    mod = importlib.import_module("test_zzz_gpu_recent_kernels")
    monkeypatch.setattr(mod, "DEV", "cpu")
    monkeypatch.setattr(mod, "_status_ok", lambda: None)
    monkeypatch.setattr(Fn, "C", KernelRestatement)
    monkeypatch.setattr(Fn, "_own_kernel_ok", lambda x: True)
    monkeypatch.setenv("TITB_TEST_STRICT", "1")          # a wrong result fails here, at once
    return mod


@pytest.mark.parametrize("name", ["sum", "mean", "max", "min"])
@pytest.mark.parametrize("shape,dim", [((7, 33, 5), 1), ((6, 40), -1), ((3, 4, 5, 6), 0), ((257,), 0)])
def test_reduce_wrappers(gpu_tests, name, shape, dim):
    gpu_tests.test_reduce_forward_backward(name, torch.float32, shape, dim)


def test_slice_split_stack_repeat_wrappers(gpu_tests):
    gpu_tests.test_slice_split_stack_repeat(torch.float32)


def test_masked_fill_and_outer_wrappers(gpu_tests):
    gpu_tests.test_masked_fill_and_outer(torch.float32)
