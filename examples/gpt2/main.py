#!/usr/bin/env python
"""GPT-2 training entry point (the reference's example/gpt2 application).

    python examples/gpt2/main.py --model gpt2 --batch_size 8 --sequence_length 1024 --synthetic
    torchrun --nproc-per-node 8 examples/gpt2/main.py --model gpt2-xl --tensor_parallel 2 \
        --pipeline_parallel 2 --num_microbatches 8 --batch_size 4 --sequence_length 1024 --synthetic
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from tinyinfinitrain_b200.cli import train_main  # noqa: E402

if __name__ == "__main__":
    sys.exit(train_main("gpt2"))
