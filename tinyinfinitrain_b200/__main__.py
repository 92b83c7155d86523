"""``python -m tinyinfinitrain_b200 <command>``:

    info                     build status, devices, measured peaks, environment switches
    build [--cpp] [-v]       compile the CUDA / C++ extensions in-tree (and the stand-alone C++ library with --cpp)
    gpt2 | llama3 [flags]    the training entry points (same flags as examples/gpt2/main.py, examples/llama3/main.py)
    kernel-bench [args]      utils.kernel_bench        fused-bench [args]   utils.fused_bench (under torchrun)
    plan [flags]             per-GPU memory plan of a model + parallel layout (utils.memory_plan)
    ab-bench [flags]         bench.py with each kernel-variant switch, one table (utils.ab_bench)
"""
from __future__ import annotations

import json
import os
import sys

SWITCHES = {
    "TITB200_ATTN": "native | sdpa: attention implementation of ops.causal_attention (sdpa = library baseline arm)",
    "TITB200_MULTIMEM": "1: NVLink kernels go through the NVSwitch multicast address (multimem) instead of peer loads / stores",
    "TITB200_SYMM_HEAP": "native: symmetric buffers from this package's own cuMem heap instead of PyTorch's",
    "TITB200_SYMM_ALLREDUCE": "1: --zero_stage 0 sums gradients with the own all-reduce kernel instead of NCCL",
    "TITB200_DETERMINISTIC": "1: sorted, atomics-free token-embedding gradient",
    "TITB200_NVTX": "1: the C++ API drops an NVTX marker per kernel dispatch (op names on an Nsight timeline)",
    "TITB200_SANITIZE": "1 (build time): ASan + UBSan build of the host C++",
    "TITB200_CXX": "host compiler for the C++ side (default /usr/bin/g++)",
    "TITB200_LLMC_DATA": "directory of the llm.c starter pack: enables the 124M logits acceptance test",
}


def info() -> int:
    import torch

    from . import _build

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = {"package": os.path.dirname(os.path.abspath(__file__)), "torch": torch.__version__, "cuda_runtime": torch.version.cuda,
           "extensions_built": _build.is_built(), "cuda_available": torch.cuda.is_available(), "devices": []}
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            out["devices"].append({"index": i, "name": p.name, "sm": f"{p.major}{p.minor}", "sms": p.multi_processor_count,
                                   "memory_gib": round(p.total_memory / 2**30, 1)})
    peaks = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(peaks):
        out["measured_peaks"] = json.load(open(peaks))
    out["switches"] = {k: {"value": os.environ.get(k, ""), "meaning": v} for k, v in SWITCHES.items()}
    print(json.dumps(out, indent=1))
    return 0


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if not argv or argv[0] in ("-h", "--help", "help"):
        print(__doc__)
        return 0
    cmd, rest = argv[0], argv[1:]
    if cmd == "info":
        return info()
    if cmd == "build":
        from . import _build

        _build.build(verbose="-v" in rest, force="-f" in rest)
        if "--cpp" in rest:
            for k, v in _build.build_cpp(verbose="-v" in rest).items():
                print(f"{k}: {v}")
        return 0
    if cmd in ("gpt2", "llama3"):
        from .cli import train_main

        sys.argv = [f"tinyinfinitrain_b200 {cmd}"] + rest
        return train_main(cmd)
    if cmd == "ab-bench":
        from .utils import ab_bench

        return ab_bench.main(rest)
    if cmd == "plan":
        from .utils import memory_plan

        return memory_plan.main(rest)
    if cmd in ("kernel-bench", "fused-bench"):
        from .utils import fused_bench, kernel_bench

        sys.argv = [cmd] + rest
        (kernel_bench if cmd == "kernel-bench" else fused_bench).main()
        return 0
    print(f"unknown command {cmd!r}\n{__doc__}")
    return 2


if __name__ == "__main__":
    sys.exit(main())
