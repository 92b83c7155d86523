"""The memory planner's parameter arithmetic against real models, and its layout rules."""
import torch

from tinyinfinitrain_b200.models import GPT2, GPT2Config
from tinyinfinitrain_b200.models.llama3 import LLaMA3, LLaMA3Config
from tinyinfinitrain_b200.utils.memory_plan import HBM_BYTES, plan, shape_of, total_params


def _count(model):
    seen, n = set(), 0
    for p in model.parameters():
        if id(p) not in seen:
            seen.add(id(p))
            n += p.numel()
    return n


def test_parameter_counts_match_the_models():
    g = GPT2Config(block_size=64, vocab_size=300, n_layer=3, n_head=4, n_embd=64)
    assert total_params(shape_of(g)) == _count(GPT2(g))
    l = LLaMA3Config(block_size=64, vocab_size=384, n_layer=2, n_head=8, n_kv_head=2, n_embd=64, ffn_dim=192)
    assert total_params(shape_of(l)) == _count(LLaMA3(l))
    assert total_params(shape_of("gpt2")) == 124_475_904          # llm.c's count for the padded 124M model
    assert total_params(shape_of("llama3-8b")) == 8_030_261_248


def test_single_rank_plan_counts_every_parameter_once():
    g = GPT2Config(block_size=64, vocab_size=300, n_layer=3, n_head=4, n_embd=64)
    p = plan(g, batch=2, seq=64)
    assert p["parameters_on_rank"] == _count(GPT2(g))
    b = p["bytes"]
    assert b["parameters_bf16"] == 2 * p["parameters_on_rank"] and b["main_gradients_fp32"] == 4 * p["parameters_on_rank"]
    assert b["optimizer_state_fp32"] == 12 * p["parameters_on_rank"]
    assert b["total"] == sum(v for k, v in b.items() if k != "total")


def test_layout_rules():
    one = plan("gpt2", dp=1)
    eight = plan("gpt2", dp=8)
    assert eight["bytes"]["optimizer_state_fp32"] * 8 == one["bytes"]["optimizer_state_fp32"]   # ZeRO-1 shards the state
    assert plan("gpt2", dp=8, zero_stage=0)["bytes"]["optimizer_state_fp32"] == one["bytes"]["optimizer_state_fp32"]
    assert eight["bytes"]["parameters_bf16"] == one["bytes"]["parameters_bf16"]                  # parameters stay replicated
    tp1, tp4 = plan("llama3-8b", tp=1, batch=1, seq=4096), plan("llama3-8b", tp=4, batch=1, seq=4096)
    assert tp4["parameters_on_rank"] < tp1["parameters_on_rank"] / 3.9                            # matrices split, norms not
    assert tp4["parameters_on_rank"] > tp1["parameters_on_rank"] / 4
    # pipeline: layers split, the first stage keeps more micro-batches in flight than the last
    st = [plan("gpt2-xl", tp=2, pp=2, dp=2, batch=4, seq=1024, micro_batches=8, stage=s) for s in range(2)]
    assert st[0]["layers_on_stage"] + st[1]["layers_on_stage"] == 48
    assert st[0]["bytes"]["activations"] == 2 * st[1]["bytes"]["activations"]
    assert st[1]["bytes"]["logits"] > 0 and st[0]["bytes"]["logits"] == 0
    # the configurations this framework is benchmarked on fit a B200 with room to spare
    for cfg in (dict(model="gpt2", dp=8), dict(model="llama3-1b", tp=8, batch=4, seq=2048),
                dict(model="llama3-8b", tp=4, dp=2, batch=2, seq=4096)):
        p = plan(**cfg)
        assert p["fits_b200"] and p["bytes"]["total"] < HBM_BYTES


def test_cli(capsys):
    from tinyinfinitrain_b200.__main__ import main
    assert main(["plan", "--model", "llama3-1b", "--tp", "8", "--batch", "4", "--seq", "2048"]) == 0
    out = capsys.readouterr().out
    assert '"fits_b200": true' in out and '"tp": 8' in out
