"""Hugging Face checkpoints -> this package's models (GPT-2 Conv1D transposition, LLaMA q/k/v and gate/up fusion):
a randomly initialised HF model saved to a directory and opened with FromPretrained gives the same logits."""
import pytest
import torch

from tinyinfinitrain_b200.models import GPT2, LLaMA3

transformers = pytest.importorskip("transformers")


def test_gpt2_from_pretrained_directory(tmp_path):
    from transformers import GPT2Config as HC, GPT2LMHeadModel

    torch.manual_seed(0)
    hf = GPT2LMHeadModel(HC(vocab_size=211, n_positions=32, n_embd=48, n_layer=2, n_head=4,
                            activation_function="gelu_new", resid_pdrop=0.0, embd_pdrop=0.0, attn_pdrop=0.0)).eval()
    hf.save_pretrained(tmp_path / "g")
    ours = GPT2.FromPretrained(str(tmp_path / "g"))
    assert ours.config.vocab_size == 211 and ours.config.padded_vocab_size % 128 == 0
    idx = torch.randint(0, 211, (2, 32), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        assert torch.allclose(ours(idx), hf(input_ids=idx).logits, atol=2e-4, rtol=1e-4)


def test_llama_from_pretrained_directory(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM

    torch.manual_seed(0)
    kw = dict(vocab_size=300, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=8,
              num_key_value_heads=4, max_position_embeddings=64, rms_norm_eps=1e-5, tie_word_embeddings=False)
    try:
        hc = LlamaConfig(rope_theta=500000.0, **kw)
    except TypeError:
        hc = LlamaConfig(rope_parameters={"rope_type": "default", "rope_theta": 500000.0}, **kw)
    hf = LlamaForCausalLM(hc).eval()
    hf.save_pretrained(tmp_path / "l")
    ours = LLaMA3.FromPretrained(str(tmp_path / "l"))
    assert (ours.config.n_kv_head, ours.config.rope_theta) == (4, 500000.0)
    idx = torch.randint(0, 300, (2, 40), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        assert torch.allclose(ours(idx), hf(input_ids=idx).logits, atol=2e-4, rtol=1e-4)
    with pytest.raises(AssertionError):
        GPT2.FromPretrained(str(tmp_path / "l"))
