"""Utilities: training-step driver, llm.c file formats, checkpoints, timers and metrics."""
from . import llmc  # noqa: F401
from .checkpoint import load_checkpoint, save_checkpoint  # noqa: F401
from .profiling import (CudaTimer, JsonlLogger, PhaseProfiler, ThroughputMeter, annotate_modules, nvtx_range,  # noqa: F401
                        torch_profile)
from .train import ParallelTrainStep, TrainStep  # noqa: F401
