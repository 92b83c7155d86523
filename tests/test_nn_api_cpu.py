"""Python ``nn`` layer with the reference's names: modules, containers, ``nn.function`` helpers and ``nn.init``
(reference: infini_train/include/nn/**, src/nn/**)."""
import math

import pytest
import torch

from tinyinfinitrain_b200 import nn
from tinyinfinitrain_b200.nn import functional as F
from tinyinfinitrain_b200.nn import init


def test_linear_reset_matches_the_reference_recipe():
    init.manual_seed(1)
    lin = nn.Linear(300, 40)
    assert lin.type() == "Linear" and tuple(lin.weight.shape) == (40, 300) and tuple(lin.bias.shape) == (40,)
    # KaimingUniform(a = sqrt(5)) over fan_in 300: bound = sqrt(3) * sqrt(2 / (1 + 5)) / sqrt(300) = 1 / sqrt(300)
    bound = 1.0 / math.sqrt(300)
    assert float(lin.weight.abs().max()) <= bound and float(lin.weight.abs().max()) > 0.9 * bound
    assert float(lin.bias.abs().max()) <= bound
    assert init.CalculateFanInAndFanOut(torch.empty(40, 300)) == (300, 40)
    assert init.CalculateFanInAndFanOut(torch.empty(8, 4, 3, 3)) == (36, 72)
    with pytest.raises(ValueError):
        init.CalculateFanInAndFanOut(torch.empty(5))
    assert nn.Linear(4, 3, bias=False).bias is None


def test_init_functions_are_seeded_and_shaped():
    a, b = torch.empty(1000), torch.empty(1000)
    init.Normal(a, 1.0, 2.0, generator=7)
    init.Normal(b, 1.0, 2.0, generator=7)
    assert torch.equal(a, b) and abs(float(a.mean()) - 1.0) < 0.3 and abs(float(a.std()) - 2.0) < 0.3
    init.Uniform(a, -3.0, -1.0, generator=7)
    assert float(a.min()) >= -3.0 and float(a.max()) < -1.0
    assert float(init.Ones(torch.empty(3)).sum()) == 3.0 and float(init.Zeros(torch.ones(3)).sum()) == 0.0
    assert init.Arange(2, 6).tolist() == [2, 3, 4, 5] and init.Arange(0, 3).dtype == torch.int64
    emb = nn.Embedding(50, 8)
    assert abs(float(emb.weight.std()) - 1.0) < 0.25           # Normal(0, 1)
    ln = nn.LayerNorm(8)
    assert float(ln.weight.sum()) == 8.0 and float(ln.bias.abs().sum()) == 0.0


def test_containers_and_state_dict_names():
    blocks = nn.Sequential(nn.Linear(4, 4), nn.Sigmoid(), nn.Linear(4, 2))
    tr = nn.ModuleDict({"wte": nn.Embedding(10, 4), "h": blocks, "ln_f": nn.LayerNorm(4)})

    class Net(nn.Module):
        kType = "Net"

        def __init__(self):
            super().__init__()
            self.transformer = tr
            self.head = nn.Linear(4, 10, bias=False)
            self.head.weight = tr["wte"].weight        # tied

    net = Net()
    assert net.type() == "Net" and blocks.type() == "Sequential" and tr.type() == "ModuleDict"
    sd = net.StateDict()
    assert set(sd) == {"transformer.wte.weight", "transformer.h.0.weight", "transformer.h.0.bias", "transformer.h.2.weight",
                       "transformer.h.2.bias", "transformer.ln_f.weight", "transformer.ln_f.bias", "head.weight"}
    assert sd["head.weight"] is sd["transformer.wte.weight"]
    assert len(net.Parameters()) == 7                           # the tied tensor is listed once
    assert net.To("cpu").head.weight is net.transformer["wte"].weight
    assert len(blocks) == 3 and blocks[1].type() == "Sigmoid" and "h" in tr and list(tr.keys()) == ["wte", "h", "ln_f"]
    with pytest.raises(RuntimeError, match="Not implemented"):
        tr(torch.zeros(1))
    seen = []
    net.Apply(lambda m: seen.append(m.type()))
    assert seen[-1] == "Net" and seen.index("Linear") < seen.index("Sequential")      # children first
    assert net.has_parameter("nope") is False and net.head.has_parameter("weight")
    y = blocks(torch.randn(3, 4))
    assert tuple(y.shape) == (3, 2)
    out = net.head.Forward([torch.randn(2, 4)])
    assert isinstance(out, list) and tuple(out[0].shape) == (2, 10)


def test_function_namespace_matches_torch():
    x = torch.randn(3, 4, 5).abs() + 0.5
    assert torch.equal(F.Tril(x[0]), torch.tril(x[0])) and torch.equal(F.Triu(x[0], 1), torch.triu(x[0], 1))
    assert torch.equal(F.Ones([2, 3]), torch.ones(2, 3))
    for name, ref in (("Reciprocal", torch.reciprocal), ("Sin", torch.sin), ("Cos", torch.cos), ("Tanh", torch.tanh),
                      ("Rsqrt", torch.rsqrt), ("Sigmoid", torch.sigmoid)):
        assert torch.allclose(getattr(F, name)(x), ref(x), atol=1e-6), name
    assert torch.allclose(F.Pow(x, 3.0), x ** 3) and torch.allclose(F.Pow(2.0, x), 2.0 ** x)
    assert torch.allclose(F.Mean(x, 1), x.mean(1)) and torch.allclose(F.Mean(x, 2, True), x.mean(2, keepdim=True))
    assert torch.allclose(F.Sum(x, 0), x.sum(0)) and torch.equal(F.Max(x, 1), x.amax(1)) and torch.equal(F.Min(x, -1), x.amin(-1))
    assert torch.allclose(F.Softmax(x, 1), torch.softmax(x, 1), atol=1e-6)
    assert torch.equal(F.Slice(x, [0, 1, 0], [3, 4, 5], [1, 2, 2]), x[0:3, 1:4:2, 0:5:2])
    assert torch.equal(F.Stack([x, x + 1], 1), torch.stack([x, x + 1], 1))
    loss = nn.CrossEntropyLoss()(torch.randn(6, 9), torch.randint(0, 9, (6,)))
    assert loss.dim() == 0 and float(loss) > 0
