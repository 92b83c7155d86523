#!/usr/bin/env python
"""LLaMA-3 training entry point.

    torchrun --nproc-per-node 8 examples/llama3/main.py --model llama3-1b --tensor_parallel 8 \
        --batch_size 4 --sequence_length 2048 --synthetic
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tinyinfinitrain_b200.cli import train_main  # noqa: E402

if __name__ == "__main__":
    sys.exit(train_main("llama3"))
