"""The A/B driver: candidate parsing, result parsing, the table, failure handling (stand-in runner) and one real
pass over bench.py's CPU dry run."""
import json
import subprocess
from types import SimpleNamespace

from tinyinfinitrain_b200.utils import ab_bench


def test_candidate_and_result_parsing():
    assert ab_bench.split_candidate("A=1") == ({"A": "1"}, [])
    assert ab_bench.split_candidate("A=1 B=x --dp_buckets 4") == ({"A": "1", "B": "x"}, ["--dp_buckets", "4"])
    out = 'noise\n{"not": "it"}\n{"metric": "m", "value": 5.0, "ms_per_step": 2.0, "config": {"final_loss": 1.5}}\ntrailer'
    assert ab_bench.parse_result(out)["value"] == 5.0 and ab_bench.parse_result("nothing") is None
    cmd = ab_bench.bench_command(4, 3, 2, ["--x"], 1234)
    assert "torch.distributed.run" in cmd and "--nproc-per-node=4" in cmd and cmd[-1] == "--x"
    assert ab_bench.bench_command(1, 3, 2, [], 1)[1] == "bench.py"


def test_table_and_failures_with_a_stand_in_runner(capsys, tmp_path):
    calls = []

    def runner(cmd, cwd, env, capture_output, text, timeout):
        calls.append({k: v for k, v in env.items() if k.startswith("TITB200_")})
        if env.get("TITB200_BROKEN") == "1":
            return SimpleNamespace(returncode=1, stdout="", stderr="Traceback\nRuntimeError: kernel says no")
        if env.get("TITB200_SLOW") == "1":
            raise subprocess.TimeoutExpired(cmd, timeout)
        v = 1100.0 if env.get("TITB200_FAST") == "1" else 1000.0
        return SimpleNamespace(returncode=0, stderr="", stdout=json.dumps(
            {"value": v, "ms_per_step": 1e3 / v, "config": {"final_loss": 2.0, "kernel_status": 0}, "e2e": {"value": v}}))

    out = tmp_path / "ab.json"
    rc = ab_bench.main(["--only", "TITB200_FAST=1", "TITB200_BROKEN=1", "TITB200_SLOW=1", "TITB200_OTHER=2", "--json_out", str(out)],
                       runner=runner)
    assert rc == 0
    text = capsys.readouterr().out
    assert "1.100" in text and "kernel says no" in text and "no result within" in text
    rows = json.load(open(out))
    assert [r["ok"] for r in rows] == [True, True, False, False, True, True]
    assert rows[-1]["env"] == {"TITB200_FAST": "1", "TITB200_OTHER": "2"}        # only what ran goes into the combined run
    assert calls[0] == {}                                                          # the default run carries no switch


def test_real_dry_run_on_cpu(capsys):
    rc = ab_bench.main(["--steps", "2", "--warmup", "3", "--only", "TITB200_DETERMINISTIC=1", "--no_combined",
                        "--bench_args", "--device", "cpu", "--tiny", "--batch", "2", "--seq", "32"])
    text = capsys.readouterr().out
    assert rc == 0 and "TITB200_DETERMINISTIC=1" in text and "failed" not in text
