"""The C++ API without Python at run time: builds libtitb200_framework.so, the C++ test program (the reference's gtest
cases restated in C++: tests/cpp/facade_api_test.cc) and the C++ training example, and runs both on the CPU."""
import subprocess

import pytest
import torch

from tinyinfinitrain_b200 import _build
from tinyinfinitrain_b200._lib import C


@pytest.fixture(scope="module")
def built():
    return _build.build_cpp()


def test_cpp_api_program_passes_on_cpu(built, tmp_path):
    r = subprocess.run([str(built["facade_api_test"]), "cpu", str(tmp_path)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "all checks passed" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


def test_cpp_training_example_runs_and_generates(built, tmp_path):
    toks = torch.randint(0, 50257, (3000,), generator=torch.Generator().manual_seed(0))
    C.llmc_write_tokens(str(tmp_path / "t.bin"), toks, 20240520)
    C.write_tokenizer(str(tmp_path / "tok.bin"), [f"<{i}>".encode() for i in range(50257)], 20240328, 50256)
    r = subprocess.run([str(built["train_gpt2"]), "--input_bin", str(tmp_path / "t.bin"), "--tokenizer_bin",
                        str(tmp_path / "tok.bin"), "--device", "cpu", "--n_layer", "1", "--n_head", "2", "--n_embd", "32",
                        "--sequence_length", "16", "--total_batch_size", "64", "--num_iteration", "3",
                        "--freq_generate_txt", "2", "--text_length", "8", "--learning_rate", "0.05"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    losses = [float(line.split("loss")[1]) for line in r.stdout.splitlines() if line.startswith("step")]
    assert len(losses) == 4 and losses[-1] < losses[0]          # num_iteration + 1 steps on the same two batches
    assert r.stdout.count("The meaning of life is<") == 2
