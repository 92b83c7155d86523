#!/usr/bin/env python
"""Fetches the llm.c starter pack (GPT-2 124M weights in fp32 and bf16, the debug state, the GPT-2 tokenizer and
the TinyShakespeare token files) into ``<dest>/`` with the token files under ``<dest>/tinyshakespeare/`` -- the
layout the reference's tests expect under ``Data/`` (its download_starter_pack.sh:7-24).  Needs network access.

    python examples/fetch_starter_pack.py --dest Data
    TITB200_LLMC_DATA=Data python -m pytest tests/test_logits_blob.py      # the 124M logits acceptance check
    python examples/gpt2/main.py --llmc_filepath Data/gpt2_124M.bin \\
        --input_bin Data/tinyshakespeare/tiny_shakespeare_train.bin --tokenizer_bin Data/gpt2_tokenizer.bin

The logits blob ``gpt2_logits_reference.bin`` is not part of the pack: copy it from the reference project's
``Data/`` directory into ``<dest>/``.
"""
from __future__ import annotations

import argparse
import os
import sys
import urllib.request

BASE_URL = "https://huggingface.co/datasets/karpathy/llmc-starter-pack/resolve/main/"
FILES = ["gpt2_124M.bin", "gpt2_124M_bf16.bin", "gpt2_124M_debug_state.bin", "gpt2_tokenizer.bin",
         "tiny_shakespeare_train.bin", "tiny_shakespeare_val.bin"]


def target_path(dest: str, name: str) -> str:
    sub = "tinyshakespeare" if name.startswith("tiny_shakespeare") else ""
    return os.path.join(dest, sub, name)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dest", default="Data")
    ap.add_argument("--force", action="store_true", help="download again even if the file exists")
    args = ap.parse_args(argv)
    os.makedirs(os.path.join(args.dest, "tinyshakespeare"), exist_ok=True)
    failed = 0
    for name in FILES:
        path = target_path(args.dest, name)
        if os.path.exists(path) and not args.force:
            print(f"have {path}")
            continue
        print(f"downloading {name} ...", flush=True)
        try:
            urllib.request.urlretrieve(f"{BASE_URL}{name}?download=true", path + ".part")
            os.replace(path + ".part", path)
        except Exception as e:  # noqa: BLE001 - report and continue with the other files
            print(f"  failed: {e}", file=sys.stderr)
            failed += 1
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
