"""The C++ facade's LLaMA-3 (csrc/core/framework/llama3.cc: RMSNorm, Rope, grouped-query attention through
RepeatInterleave, SwiGLU) against the Python model: same-seed initialisation, llm.c-style checkpoint round trip,
logits, loss and gradients; and the three Functions it adds against PyTorch autograd."""
import torch

from tinyinfinitrain_b200 import ops
from tinyinfinitrain_b200._lib import C
from tinyinfinitrain_b200.models import LLaMA3, LLaMA3Config


def test_rope_swiglu_rmsnorm_functions_match_autograd():
    torch.manual_seed(0)
    x0 = torch.randn(2, 5, 3, 8)
    x = C.FwTensor(x0.clone(), True)
    y = C.fw_function("Rope", [10000.0, 2]).Apply([x])[0]
    xr = x0.clone().requires_grad_(True)
    ref = ops.rope_ref(xr, 2, 10000.0)
    g = torch.randn_like(ref)
    y.Backward(C.FwTensor(g.clone()))
    ref.backward(g)
    assert torch.allclose(y.torch(), ref, atol=1e-6) and torch.allclose(x.grad().torch(), xr.grad, atol=1e-6)

    z0 = torch.randn(4, 12)
    z = C.FwTensor(z0.clone(), True)
    s = C.fw_function("SwiGLU").Apply([z])[0]
    zr = z0.clone().requires_grad_(True)
    sr = torch.nn.functional.silu(zr[:, :6]) * zr[:, 6:]
    g = torch.randn_like(sr)
    s.Backward(C.FwTensor(g.clone()))
    sr.backward(g)
    assert torch.allclose(s.torch(), sr, atol=1e-6) and torch.allclose(z.grad().torch(), zr.grad, atol=1e-6)

    w0 = torch.rand(12) + 0.5
    xx, ww = C.FwTensor(z0.clone(), True), C.FwTensor(w0.clone(), True)
    r = C.fw_function("RMSNorm", [1e-5]).Apply([xx, ww])[0]
    a, b = z0.clone().requires_grad_(True), w0.clone().requires_grad_(True)
    rr = ops.rmsnorm_ref(a, b, 1e-5)
    g = torch.randn_like(rr)
    r.Backward(C.FwTensor(g.clone()))
    rr.backward(g)
    assert torch.allclose(r.torch(), rr, atol=1e-6)
    assert torch.allclose(xx.grad().torch(), a.grad, atol=1e-5) and torch.allclose(ww.grad().torch(), b.grad, atol=1e-5)


def test_cpp_llama3_matches_python_model(tmp_path):
    cfg = LLaMA3Config(block_size=32, vocab_size=200, n_layer=2, n_head=8, n_kv_head=2, n_embd=64, ffn_dim=96)
    same_seed = C.FwLLaMA3(32, 200, 2, 8, 2, 64, 96)
    py = LLaMA3(cfg, seed=42)
    sd = same_seed.StateDict()
    assert set(sd) == set(py.StateDict())
    assert all(torch.equal(sd[k].torch(), v) for k, v in py.StateDict().items())       # same seed, same weights

    with torch.no_grad():
        for n, p in py.named_parameters():
            if "ln_" in n:
                p.add_(0.1 * torch.randn_like(p))
    path = str(tmp_path / "llama.bin")
    py.SaveLLMC(path)
    cpp = C.FwLLaMA3.FromLLMC(path)
    g = torch.Generator().manual_seed(1)
    idx, tgt = torch.randint(0, 200, (2, 24), generator=g), torch.randint(0, 200, (2, 24), generator=g)
    logits = cpp.Forward([C.FwTensor(idx)])[0]
    ref = py(idx)
    assert torch.allclose(logits.torch(), ref, atol=1e-5)
    loss = C.FwCrossEntropyLoss().Forward([logits, C.FwTensor(tgt)])[0]
    loss.Backward()
    ref_loss = torch.nn.functional.cross_entropy(ref.reshape(-1, 200), tgt.reshape(-1))
    ref_loss.backward()
    assert abs(float(loss.torch().detach()) - float(ref_loss)) < 1e-5
    for name in ("transformer.h.0.attn.c_attn.weight", "transformer.h.1.mlp.c_fc.weight", "transformer.ln_f.weight",
                 "transformer.wte.weight", "lm_head.weight"):
        assert torch.allclose(cpp.StateDict()[name].grad().torch(), py.StateDict()[name].grad, atol=1e-5), name


def test_causal_attention_function_matches_reference_math():
    torch.manual_seed(0)
    B, T, Hq, Hkv, hd = 2, 9, 4, 2, 8
    q0, k0, v0 = torch.randn(B, T, Hq, hd), torch.randn(B, T, Hkv, hd), torch.randn(B, T, Hkv, hd)
    q, k, v = (C.FwTensor(t.clone(), True) for t in (q0, k0, v0))
    o = C.fw_function("CausalAttention").Apply([q, k, v])[0]
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q0, k0, v0))
    ref = ops.attention_ref(qr, kr, vr)
    g = torch.randn_like(ref)
    o.Backward(C.FwTensor(g.clone()))
    ref.backward(g)
    assert torch.allclose(o.torch(), ref, atol=1e-6)
    for a, b in ((q, qr), (k, kr), (v, vr)):
        assert torch.allclose(a.grad().torch(), b.grad, atol=1e-5)


def test_module_cast_to_bfloat16_keeps_ties_and_runs():
    m = C.FwGPT2(16, 97, 2, 2, 32)
    idx = torch.randint(0, 97, (2, 16), generator=torch.Generator().manual_seed(0))
    ref = m.Forward([C.FwTensor(idx)])[0].torch()
    m.ToDtype("bfloat16")
    sd = m.StateDict()
    assert all(t.Dtype() == "bfloat16" for t in sd.values())
    assert sd["lm_head.weight"].torch().data_ptr() == sd["transformer.wte.weight"].torch().data_ptr()
    out = m.Forward([C.FwTensor(idx)])[0].torch()
    assert out.dtype == torch.bfloat16 and (out.float() - ref).abs().max() < 2e-2
