"""The C++ facade (reference class names) on cuda:0 against the same facade on the CPU, and the C++ API test program."""
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



def _fw(t, dev, requires_grad=False):
    ft = C.FwTensor(t.clone(), requires_grad)
    return ft.To(dev) if dev != "cpu" else ft


def _facade_run(dev):
    """A tour through the C++ facade's view-like, reduction and mask Functions; returns every result as CPU tensors."""
    torch.manual_seed(8)
    out = {}
    x0 = torch.randn(3, 4, 6)
    x = _fw(x0, dev, True)
    parts = x.Split(2, 2)                                            # Split (multi-output) -> gather kernel
    y = parts[0].Mul(parts[1]).Add(parts[2])
    y = y.Transpose(0, 1)                                            # Transpose -> gather kernel
    y = y.RepeatInterleave(2, 2)                                     # stride-0 gather / sum backward
    y = y.Slice([0, 1, 0], [4, 3, 4], [1, 1, 2])                     # Slice -> gather fwd, scatter bwd
    s = C.fw_function("Stack", [1]).Apply([y, y.MulScalar(2.0)])[0]  # Stack -> scatter fwd, gather bwd
    sm = C.fw_function("Softmax", [2]).Apply([s])[0]
    red = C.fw_function("Sum", [3, 0]).Apply([sm.Mul(s)])[0]
    red = C.fw_function("Max", [0, 1]).Apply([red])[0]
    red = C.fw_function("Mean", [2, 0]).Apply([red])[0]
    red = C.fw_function("Min", [1, 0]).Apply([red])[0]
    out["y"], out["stack"], out["softmax"], out["red"] = y.torch(), s.torch(), sm.torch(), red.torch()
    red.Backward(_fw(torch.ones(1), dev))
    out["dx"] = x.grad().torch()
    m0 = torch.tril(torch.ones(6, 6))
    a = _fw(torch.randn(2, 6, 6), dev, True)
    tri = C.fw_function("Tril", [0]).Apply([_fw(torch.ones(6, 6), dev)])[0]
    masked = a.MaskedFill(tri.Equals(0.0), -1e4)
    out["tril"], out["masked"] = tri.torch(), masked.torch()
    C.fw_function("Sum", [0, 0]).Apply([C.fw_function("Sum", [2, 0]).Apply([masked])[0]])[0].Backward(_fw(torch.ones(6), dev))
    out["da"] = a.grad().torch()
    ge_in = _fw(torch.randn(4, 9), dev, True)
    ge = C.fw_function("Gelu").Apply([ge_in])[0]                     # one kernel on the GPU
    C.fw_function("Sum", [0, 0]).Apply([C.fw_function("Sum", [1, 0]).Apply([ge])[0]])[0].Backward()
    out["gelu"], out["dgelu"] = ge.torch(), ge_in.grad().torch()
    u, v = _fw(torch.randn(5), dev, True), _fw(torch.randn(7), dev, True)
    o = u.Outer(v)
    out["outer"] = o.torch()
    C.fw_function("Sum", [0, 0]).Apply([C.fw_function("Sum", [1, 0]).Apply([o.Mul(o)])[0]])[0].Backward()
    out["du"], out["dv"] = u.grad().torch(), v.grad().torch()
    assert torch.equal(m0, out["tril"].cpu())
    return {k: t.detach().float().cpu() for k, t in out.items()}


def test_cpp_facade_cuda_ops_match_cpu_oracle():
    cpu, gpu = _facade_run("cpu"), _facade_run("cuda:0")
    for k in cpu:
        assert cpu[k].shape == gpu[k].shape, k
        tol = 2e-3 if "gelu" in k else 1e-5   # the GPU GELU uses tanh.approx
        assert torch.allclose(cpu[k], gpu[k], atol=tol, rtol=tol), k
    _status_ok()


def test_cpp_llama3_and_gpt2_on_cuda_match_the_cpu_facade():
    """The C++ models moved to cuda:0 (kernel-backed RMSNorm / Rope / SwiGLU / Gelu / LayerNorm / softmax / SGEMM and the
    gather kernel behind every transpose and slice) against the same models on the CPU."""
    g = torch.Generator().manual_seed(2)
    idx, tgt = torch.randint(0, 150, (2, 16), generator=g), torch.randint(0, 150, (2, 16), generator=g)
    for make in (lambda: C.FwLLaMA3(32, 150, 2, 4, 2, 32, 48), lambda: C.FwGPT2(32, 150, 2, 4, 32)):
        res = {}
        for dev in ("cpu", "cuda:0"):
            model = make()                       # seeded initialisation: identical weights in both runs
            if not dev.startswith("cpu"):
                model.To(dev)                    # one call on the root: parameters AND buffers (attention masks) move
                for name, t in list(model.StateDict().items()) + list(model.Buffers().items()):
                    assert "CUDA" in t.GetDevice(), (name, t.GetDevice())
            put = (lambda t: C.FwTensor(t).To(dev)) if not dev.startswith("cpu") else C.FwTensor
            logits = model.Forward([put(idx)])[0]
            loss = C.FwCrossEntropyLoss().Forward([logits, put(tgt)])[0]
            loss.Backward()
            grads = {k: v.grad().torch().float().cpu() for k, v in model.StateDict().items() if v.grad() is not None}
            res[dev] = (logits.torch().detach().float().cpu(), float(loss.torch().detach()), grads)
        assert torch.allclose(res["cpu"][0], res["cuda:0"][0], atol=2e-3, rtol=1e-3)
        assert abs(res["cpu"][1] - res["cuda:0"][1]) < 1e-3
        for k, gcpu in res["cpu"][2].items():
            assert torch.allclose(gcpu, res["cuda:0"][2][k], atol=2e-3, rtol=1e-2), k
    _status_ok()


def test_cpp_models_in_bf16_use_the_flash_attention_function():
    """C++ GPT-2 (hd 64) and LLaMA-3 (hd 64, grouped-query) cast to bf16 on cuda:0: attention runs as the fused
    CausalAttention Function (tcgen05 kernels); logits and loss stay close to the fp32 CPU model."""
    g = torch.Generator().manual_seed(3)
    idx, tgt = torch.randint(0, 300, (2, 128), generator=g), torch.randint(0, 300, (2, 128), generator=g)
    for make in (lambda: C.FwGPT2(128, 300, 2, 2, 128), lambda: C.FwLLaMA3(128, 300, 2, 4, 2, 256, 512)):
        ref_model = make()
        ref = ref_model.Forward([C.FwTensor(idx)])[0].torch()
        model = make()
        model.To("cuda:0")
        model.ToDtype("bfloat16")
        logits = model.Forward([C.FwTensor(idx).To("cuda:0")])[0]
        loss = C.FwCrossEntropyLoss().Forward([logits, C.FwTensor(tgt).To("cuda:0")])[0]
        loss.Backward()
        assert logits.torch().dtype == torch.bfloat16
        assert (logits.torch().float().cpu() - ref).abs().max() < 0.1
        grads = [v.grad().torch() for v in model.StateDict().values() if v.grad() is not None]
        assert grads and all(torch.isfinite(x.float()).all() for x in grads)
        assert any(float(x.float().abs().max()) > 0 for x in grads)
    _status_ok()


def test_cpp_api_program_passes_on_cuda(tmp_path):
    """The stand-alone C++ test program (reference gtest cases + data layer + a short GPT-2 run) on cuda:0."""
    from tinyinfinitrain_b200 import _build

    built = _build.build_cpp()
    r = subprocess.run([str(built["facade_api_test"]), "cuda", str(tmp_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "all checks passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]

