"""The CMake project for C++ users configures and knows its targets (the full build is the same sources the Python
package builds through _build.py, so this test stops after the configure step)."""
import shutil
import subprocess

import pytest
import torch


@pytest.mark.skipif(shutil.which("cmake") is None or shutil.which("nvcc") is None, reason="needs cmake and nvcc")
def test_cmake_project_configures_and_lists_its_targets(tmp_path):
    import os

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run(["cmake", "-S", root, "-B", str(tmp_path), f"-DCMAKE_PREFIX_PATH={torch.utils.cmake_prefix_path}"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    h = subprocess.run(["cmake", "--build", str(tmp_path), "--target", "help"], capture_output=True, text=True, timeout=120)
    assert h.returncode == 0, h.stderr[-2000:]
    for target in ("titb200_kernels", "titb200_framework", "train_gpt2", "facade_api_test"):
        assert target in h.stdout, target
    t = subprocess.run(["ctest", "--test-dir", str(tmp_path), "-N"], capture_output=True, text=True, timeout=120)
    assert "facade_api_cpu_matmul" in t.stdout and "facade_api_cuda_gpt2" in t.stdout
