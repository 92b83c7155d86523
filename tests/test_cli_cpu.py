"""The example entry points on CPU: one process, and gloo ranks for tensor / pipeline / data parallel layouts."""
import os
import re
import sys

import pytest

from _launch import run_group

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SMALL = ["--n_embd", "64", "--n_head", "4", "--vocab_size", "1000"]      # keeps every child process to a few seconds
COMMON = ["--device", "cpu", "--synthetic", "--num_iteration", "3", "--n_layer", "2", "--batch_size", "2",
          "--sequence_length", "16", "--dtype", "float32"] + SMALL


def _losses(out: str):
    return [float(m) for m in re.findall(r"^step \d+/\d+ \| loss ([0-9.]+)", out, flags=re.M)]


def _sane(ls, vocab):
    """Every step sees fresh random tokens, so the loss stays near ln(vocab); it must be finite and reported thrice."""
    import math

    return len(ls) == 3 and all(math.isfinite(x) and abs(x - math.log(vocab)) < 2.0 for x in ls)


def _run(cmd):
    r = run_group(cmd, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return r.stdout


@pytest.mark.parametrize("family", ["gpt2", "llama3"])
def test_single_process_training_runs(family):
    extra = [] if family == "gpt2" else ["--n_kv_head", "2", "--ffn_dim", "128"]
    out = _run([sys.executable, f"examples/{family}/main.py"] + COMMON + extra)
    assert _sane(_losses(out), 1000), out[-1500:]


@pytest.mark.parametrize("layout", [["--tensor_parallel", "2", "--pipeline_parallel", "2", "--num_microbatches", "2"],
                                    ["--tensor_parallel", "2"],                       # tp2 x dp2 with ZeRO-1
                                    ["--pipeline_parallel", "4", "--num_microbatches", "4", "--n_layer", "4"]])
def test_four_ranks_layouts(layout):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
           "127.0.0.1", "--master-port", str(29250 + os.getpid() % 200), "examples/gpt2/main.py"] + COMMON + layout
    out = _run(cmd)
    assert _sane(_losses(out), 1000), out[-1500:]


def _step_losses(out: str):
    return {int(m.group(1)): float(m.group(2)) for m in re.finditer(r"^step (\d+)/\d+ \| loss ([0-9.]+)", out, flags=re.M)}


@pytest.mark.parametrize("ranks,layout", [(1, []), (2, []), (4, ["--tensor_parallel", "2", "--zero_stage", "0"])])
def test_resume_continues_exactly_where_the_first_run_stopped(tmp_path, ranks, layout):
    """3 steps + save, then resume to 5 == 5 uninterrupted steps (same losses at steps 4 and 5), for one process,
    ZeRO-1 over two ranks, and tensor parallel x plain all-reduce data parallel over four."""
    base = [sys.executable] if ranks == 1 else \
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(ranks), "--master-addr",
         "127.0.0.1", "--master-port", str(29450 + os.getpid() % 200)]
    common = ["examples/gpt2/main.py", "--device", "cpu", "--synthetic", "--n_layer", "1", "--batch_size", "2",
              "--sequence_length", "16", "--dtype", "float32", "--learning_rate", "1e-3"] + SMALL + layout
    ck = str(tmp_path / "ck")
    full = _step_losses(_run(base + common + ["--num_iteration", "5"]))
    _run(base + common + ["--num_iteration", "3", "--save", ck])
    resumed = _step_losses(_run(base + common + ["--num_iteration", "5", "--resume", ck]))
    assert sorted(resumed) == [4, 5] and sorted(full) == [1, 2, 3, 4, 5]
    assert abs(resumed[4] - full[4]) < 1e-5 and abs(resumed[5] - full[5]) < 1e-5, (full, resumed)


def test_restart_after_failure_recipe(tmp_path):
    """Periodic checkpoints + `--resume auto`: a run that stops after step 3 of 5 (here: it was only asked for 3) is
    continued by repeating the command line, and ends where an uninterrupted run ends."""
    ck = str(tmp_path / "ck")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(29050 + os.getpid() % 40), "examples/gpt2/main.py", "--device", "cpu",
           "--synthetic", "--n_layer", "1", "--batch_size", "2", "--sequence_length", "16", "--dtype", "float32",
           "--learning_rate", "1e-3"] + SMALL + ["--save", ck, "--save_every", "1", "--resume", "auto"]
    first = _step_losses(_run(cmd + ["--num_iteration", "3"]))            # nothing to resume from yet
    assert sorted(first) == [1, 2, 3] and os.path.exists(os.path.join(ck, "optim_rank1.pt"))
    second = _step_losses(_run(cmd + ["--num_iteration", "5"]))           # same command: picks the checkpoint up
    assert sorted(second) == [4, 5]
    full = _step_losses(_run(cmd[:-4] + ["--num_iteration", "5"]))        # no --save / --resume: uninterrupted
    assert abs(second[5] - full[5]) < 1e-5


def test_multi_rank_save_writes_a_full_llmc_file_and_refuses_another_layout(tmp_path):
    """TP2 x PP2: rank 0 reassembles the full tensors from every rank's slices and writes model.bin in the llm.c layout
    (which has ONE wte: the first stage's embedding and the last stage's output projection must still be equal after
    training, or the save refuses).  Resuming the optimizer shards under another layout is refused with a clear message."""
    sys.path.insert(0, ROOT)
    ck = str(tmp_path / "ck")
    base = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4", "--master-addr",
            "127.0.0.1", "--master-port", str(29650 + os.getpid() % 200), "examples/gpt2/main.py"] + COMMON
    _run(base + ["--tensor_parallel", "2", "--pipeline_parallel", "2", "--num_microbatches", "2", "--save", ck,
                 "--learning_rate", "1e-2"])
    assert os.path.exists(os.path.join(ck, "model.bin")) and os.path.exists(os.path.join(ck, "optim_rank3.pt"))
    from tinyinfinitrain_b200.utils.llmc import load_gpt2

    m = load_gpt2(os.path.join(ck, "model.bin"))
    sd = m.StateDict()
    assert sd["transformer.wte.weight"].shape[1] == 64 and sd["transformer.h.1.mlp.c_fc.weight"].shape == (256, 64)
    assert float(sd["transformer.h.0.attn.c_attn.weight"].abs().sum()) > 0
    r = run_group(base + ["--tensor_parallel", "4", "--resume", ck, "--num_iteration", "4"], cwd=ROOT, timeout=600)
    assert r.returncode != 0 and "this job runs tp=4" in (r.stdout + r.stderr)
