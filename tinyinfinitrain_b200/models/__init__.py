"""Model zoo: GPT-2 (reference example) and LLaMA-3."""
from .gpt2 import GPT2, GPT2_PRESETS, GPT2Config  # noqa: F401
from .llama3 import LLAMA3_PRESETS, LLaMA3, LLaMA3Config  # noqa: F401
