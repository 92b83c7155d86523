"""Utilities: training-step driver, llm.c file formats, tokenizer, checkpoints, timers."""
from .train import TrainStep  # noqa: F401
