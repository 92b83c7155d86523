"""Model zoo: GPT-2 (reference example) and LLaMA-3."""
from .gpt2 import GPT2, GPT2_PRESETS, GPT2Config  # noqa: F401
