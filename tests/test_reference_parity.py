"""The reference's gtest cases restated against the C++ facade (same literals, same tolerances).

Sources: test/autograd/test_elementwise.cc:11-59, test/kernels/test_matmul.cc:12-133,
test/optimizer/test_adam.cc:11-60, test/tensor/test_tensor.cc:10-78,
test/kernels/test_dispatcher.cc:17-56 of the reference project.  The same cases run on the GPU
in test_gpu_reference_parity (marked gpu).
"""
import math
import os
import tempfile

import pytest
import torch

from tinyinfinitrain_b200._lib import C


def T(values, shape=None, dev="cpu", requires_grad=False):
    t = torch.tensor(values, dtype=torch.float32)
    if shape is not None:
        t = t.reshape(shape)
    ft = C.FwTensor(t, requires_grad)
    return ft.To(dev) if dev != "cpu" else ft


def vals(ft):
    return ft.torch().detach().cpu().flatten().tolist()


def _elementwise(dev):
    x = T([1.0, -2.0, 0.0], dev=dev)
    f = C.fw_function("Neg")
    out = f.Forward([x])
    assert vals(out[0]) == [-1.0, 2.0, -0.0]
    g = T([1.0, 1.0, 1.0], dev=dev)
    f.SetupContext([x], out)
    assert vals(f.Backward([g])[0]) == [-1.0, -1.0, -1.0]


def _matmul(dev):
    a = T([1, 2, 3, 4, 5, 6], (2, 3), dev)
    b = T([7, 8, 9, 10, 11, 12], (3, 2), dev)
    out = C.fw_function("Matmul").Forward([a, b])[0]
    assert out.Dims() == [2, 2] and vals(out) == [58, 64, 139, 154]
    a3 = T(list(range(1, 13)), (2, 2, 3), dev)
    b3 = T(list(range(1, 13)), (2, 3, 2), dev)
    out = C.fw_function("Matmul").Forward([a3, b3])[0]
    assert vals(out) == [22, 28, 49, 64, 220, 244, 301, 334]
    f = C.fw_function("Matmul")
    go = T([0.1, 0.2, 0.3, 0.4], (2, 2), dev)
    f.SetupContext([a, b], [T([0, 0, 0, 0], (2, 2), dev)])
    da, db = f.Backward([go])
    assert vals(da) == pytest.approx([2.3, 2.9, 3.5, 5.3, 6.7, 8.1], rel=1e-6)
    assert vals(db) == pytest.approx([1.3, 1.8, 1.7, 2.4, 2.1, 3.0], rel=1e-6)


def _adam(dev):
    p = T([1.0, 2.0, 3.0], dev=dev, requires_grad=True)
    grad = [0.1, -0.2, 0.3]
    lr, b1, b2, eps = 0.1, 0.9, 0.999, 1e-8
    opt = C.FwAdam([p], lr, b1, b2, eps)
    w, m, v = [1.0, 2.0, 3.0], [0.0] * 3, [0.0] * 3
    for t in range(1, 4):
        p.grad().torch().copy_(torch.tensor(grad))
        before = vals(p)
        opt.Step()
        for i in range(3):
            m[i] = b1 * m[i] + (1 - b1) * grad[i]
            v[i] = b2 * v[i] + (1 - b2) * grad[i] ** 2
            w[i] -= lr * (m[i] / (1 - b1 ** t)) / (math.sqrt(v[i] / (1 - b2 ** t)) + eps)
        assert vals(p) == pytest.approx(w, abs=1e-5)
        assert vals(p)[0] < before[0] and vals(p)[1] > before[1]   # moves against the gradient sign


def _tensor_autograd(dev):
    x = C.FwTensor(torch.tensor(2.0), False).To(dev).RequiresGrad()
    x.Pow(2).Backward()
    assert vals(x.grad()) == [4.0]
    x = T([1.0, 1.0, 1.0], dev=dev).RequiresGrad()
    y1, y2 = x.MulScalar(2.0), x.Pow(3)
    y1.Backward(T([1.0] * 3, dev=dev))
    y2.Backward(T([2.0] * 3, dev=dev))
    assert vals(x.grad()) == [8.0, 8.0, 8.0]
    t = T(list(range(1, 13)), (3, 4), dev)
    flat = t.Flatten(0, 1)
    assert flat.Dims() == [12] and vals(flat) == [float(i) for i in range(1, 13)]
    assert T([0.0] * 24, (2, 3, 4), dev).Flatten(1, -1).Dims() == [2, 12]
    tr = T([0.0] * 12, (4, 3), dev).Transpose(0, 1).Flatten(0, -1)
    assert tr.Dims() == [12] and tr.NumElements() == 12


def test_elementwise_neg():
    _elementwise("cpu")


def test_matmul_forward_batched_backward():
    _matmul("cpu")


def test_adam_three_steps_closed_form():
    _adam("cpu")


def test_tensor_backward_and_flatten():
    _tensor_autograd("cpu")


def test_dispatcher_register_call_errors():
    r = C.fw_dispatcher_selftest()
    assert r["void_called"] and r["int_result"] == 5 and r["separate_device_keys"]
    with pytest.raises(RuntimeError, match="Kernel already registered"):
        C.fw_dispatcher_register_duplicate()
    with pytest.raises(RuntimeError, match="Kernel not found"):
        C.fw_dispatcher_get_missing()
    assert r["has_linear_cpu"] and r["has_adam_cuda"]


def test_function_graph_matches_torch_autograd():
    """A small graph through many op Functions: gradients equal PyTorch's."""
    torch.manual_seed(0)
    a0, b0 = torch.randn(4, 6), torch.rand(6) + 0.5
    a, b = C.FwTensor(a0, True), C.FwTensor(b0, True)
    y = a.Mul(b).Tanh().Add(a.Div(b)).Sin()
    z = C.fw_function("Sum", [1, 0]).Apply([y])[0]
    w = C.fw_function("Mean", [0, 0]).Apply([z])[0]
    w.Backward()
    at, bt = a0.clone().requires_grad_(True), b0.clone().requires_grad_(True)
    (torch.sin(torch.tanh(at * bt) + at / bt)).sum(1).mean(0).backward()
    assert torch.allclose(a.grad().torch(), at.grad, atol=1e-5)
    assert torch.allclose(b.grad().torch(), bt.grad, atol=1e-5)
    # Split is multi-output: it fires once both halves delivered their gradient
    x = C.FwTensor(torch.arange(8.0).reshape(2, 4), True)
    lo, hi = x.Split(2, 1)
    lo.MulScalar(2.0).Add(hi.MulScalar(3.0)).Backward(C.FwTensor(torch.ones(2, 2)))
    assert vals(x.grad()) == [2, 2, 3, 3, 2, 2, 3, 3]


def test_modules_linear_layernorm_crossentropy_sgd():
    torch.manual_seed(1)
    lin = C.FwLinear(5, 3)
    ln = C.FwLayerNorm(3)
    loss_fn = C.FwCrossEntropyLoss()
    x = C.FwTensor(torch.randn(2, 4, 5))
    tgt = C.FwTensor(torch.randint(0, 3, (2, 4)))
    h = ln.Forward(lin.Forward([x]))[0]
    loss = loss_fn.Forward([h, tgt])[0]
    loss.Backward()
    w = lin.parameter("weight")
    tl = torch.nn.Linear(5, 3)
    with torch.no_grad():
        tl.weight.copy_(w.torch()); tl.bias.copy_(lin.parameter("bias").torch())
    ref = torch.nn.functional.cross_entropy(
        torch.nn.functional.layer_norm(tl(x.torch()), (3,)).reshape(-1, 3), tgt.torch().reshape(-1))
    ref.backward()
    assert abs(vals(loss)[0] - ref.item()) < 1e-5
    assert torch.allclose(w.grad().torch(), tl.weight.grad, atol=1e-5)
    before = w.torch().clone()
    opt = C.FwSGD(lin.Parameters(), 0.1)
    opt.Step()
    assert torch.allclose(w.torch(), before - 0.1 * tl.weight.grad, atol=1e-6)
    opt.ZeroGrad()
    assert w.grad().torch().abs().sum().item() == 0
    sd = C.FwSequential([lin, ln]).StateDict()
    assert set(sd) == {"0.weight", "0.bias", "1.weight", "1.bias"}


def test_cpp_gpt2_matches_python_model_and_llmc_roundtrip():
    from tinyinfinitrain_b200.models import GPT2, GPT2Config

    cfg = GPT2Config(block_size=32, vocab_size=120, n_layer=2, n_head=2, n_embd=32)
    py = GPT2(cfg)
    path = os.path.join(tempfile.mkdtemp(), "m.bin")
    py.SaveLLMC(path)
    cpp = C.FwGPT2.FromLLMC(path)
    keys = set(cpp.StateDict())
    assert "transformer.h.1.attn.c_attn.weight" in keys and "lm_head.weight" in keys and "transformer.wte.weight" in keys
    assert len(cpp.Parameters()) == len(list(py.parameters()))     # the tied tensor is listed once
    idx = torch.randint(0, 120, (2, 16))
    logits = cpp.Forward([C.FwTensor(idx)])[0].torch()
    assert torch.allclose(logits, py(idx), atol=2e-4)
    # same seed => same initial weights as the Python model (std::mt19937(42) + normal_distribution<float>)
    fresh = C.FwGPT2(32, 120, 2, 2, 32)
    assert torch.allclose(fresh.StateDict()["transformer.h.0.attn.c_attn.weight"].torch(),
                          py.StateDict()["transformer.h.0.attn.c_attn.weight"])


def test_attention_masks_are_buffers_of_the_module_tree():
    """The causal masks are registered buffers (the reference's "bias"), reachable from the root by dotted name, so the
    recursive Module::To(Device) moves them together with the parameters (the move itself is checked on a GPU)."""
    from tinyinfinitrain_b200._lib import C

    for model, layers in ((C.FwGPT2(16, 50, 2, 2, 16), 2), (C.FwLLaMA3(16, 50, 3, 2, 1, 16, 24), 3)):
        bufs = model.Buffers()
        names = sorted(k for k in bufs if k.endswith(".attn.bias"))
        assert len(names) == layers, names
        for k in names:
            m = bufs[k].torch()
            assert m.shape == (16, 16) and torch.equal(m, torch.triu(torch.ones(16, 16), 1))
            assert "CPU" in bufs[k].GetDevice()
        assert not any(k.endswith(".attn.bias") for k in model.StateDict())   # buffers are not parameters


def test_save_as_npy_and_print(tmp_path):
    import numpy as np

    t = C.FwTensor(torch.arange(6.0).reshape(2, 3))
    p = str(tmp_path / "t.npy")
    t.SaveAsNpy(p)
    assert np.array_equal(np.load(p), np.arange(6.0, dtype=np.float32).reshape(2, 3))
    assert "tensor([[0.0000, 1.0000, 2.0000]," in repr(t)


@pytest.mark.gpu
def test_gpu_reference_parity():
    for fn in (_elementwise, _matmul, _adam, _tensor_autograd):
        fn("cuda:0")
