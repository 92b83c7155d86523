"""A/B driver for the kernel variants that are selected through environment switches.

    python -m tinyinfinitrain_b200.utils.ab_bench --steps 20 --warmup 5 --json_out ab.json
    python -m tinyinfinitrain_b200.utils.ab_bench --gpus 8 --only TITB200_NO_MULTIMEM=1 "--dp_buckets 4"

Runs ``bench.py`` once with the defaults and once per candidate (one switch at a time, then all of them together),
each as its own process with a time limit, and prints one table: tokens/s, ms per step, ratio to the default run,
final loss and the kernel status word.  A candidate is an environment assignment (``NAME=value``) or, when it starts
with ``--``, extra ``bench.py`` flags.  Nothing is changed permanently; the table is the evidence for flipping a
default in the source.  Multi-GPU runs go through ``torch.distributed.run`` on 127.0.0.1.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from typing import Dict, List, Optional

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

# Candidates when --only is not given: the switches / flags that still select a non-default variant.
DEFAULT_CANDIDATES = [
    "TITB200_DETERMINISTIC=1",
]


def bench_command(gpus: int, steps: int, warmup: int, extra: List[str], port: int) -> List[str]:
    tail = ["bench.py", "--gpus", str(gpus), "--steps", str(steps), "--warmup", str(warmup)] + extra
    if gpus == 1:
        return [sys.executable] + tail
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={gpus}", "--master-addr", "127.0.0.1",
            "--master-port", str(port)] + tail


def parse_result(stdout: str) -> Optional[Dict]:
    """The last line of ``stdout`` that is a JSON object with a ``value`` key."""
    for line in reversed(stdout.splitlines()):
        line = line.strip()
        if line.startswith("{") and line.endswith("}"):
            try:
                rec = json.loads(line)
            except ValueError:
                continue
            if "value" in rec:
                return rec
    return None


def split_candidate(cand: str):
    """``NAME=value [NAME2=value2 ...]`` -> environment; anything from the first ``--`` on -> bench.py flags."""
    env, flags = {}, []
    for tok in cand.split():
        if flags or tok.startswith("--"):
            flags.append(tok)
        elif "=" in tok:
            k, v = tok.split("=", 1)
            env[k] = v
        else:
            raise ValueError(f"candidate token {tok!r} is neither NAME=value nor a --flag")
    return env, flags


def run_one(label: str, env_add: Dict[str, str], flags: List[str], a, port: int, runner=subprocess.run) -> Dict:
    env = {k: v for k, v in os.environ.items() if not k.startswith("TITB200_") or k in ("TITB200_CXX", "TITB200_LLMC_DATA")}
    env.update(env_add)
    cmd = bench_command(a.gpus, a.steps, a.warmup, a.bench_args + flags, port)
    try:
        r = runner(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=a.timeout)
        rec = parse_result(r.stdout) if r.returncode == 0 else None
        err = "" if rec else (r.stderr or r.stdout)[-400:]
    except subprocess.TimeoutExpired:
        rec, err = None, f"no result within {a.timeout} s"
    out = {"label": label, "env": env_add, "flags": flags, "ok": rec is not None}
    if rec:
        cfg = rec.get("config", {})
        out.update(value=rec["value"], ms_per_step=rec.get("ms_per_step"), e2e=rec.get("e2e", {}).get("value"),
                   final_loss=cfg.get("final_loss"), kernel_status=cfg.get("kernel_status"), clocks=rec.get("clocks"))
    else:
        out["error"] = err
    return out


def table(rows: List[Dict]) -> str:
    base = next((r for r in rows if r["label"] == "default" and r["ok"]), None)
    lines = [f"{'run':<44} {'tokens/s':>12} {'ms/step':>9} {'vs default':>10} {'loss':>8} {'status':>6}"]
    for r in rows:
        if not r["ok"]:
            lines.append(f"{r['label']:<44} {'failed: ' + r['error'].strip().splitlines()[-1][:60] if r.get('error') else 'failed'}")
            continue
        ratio = f"{r['value'] / base['value']:.3f}" if base else "-"
        loss = f"{r['final_loss']:.3f}" if isinstance(r.get("final_loss"), (int, float)) else "-"
        lines.append(f"{r['label']:<44} {r['value']:>12.0f} {r['ms_per_step']:>9.3f} {ratio:>10} {loss:>8} {str(r.get('kernel_status')):>6}")
    return "\n".join(lines)


def main(argv=None, runner=subprocess.run) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--timeout", type=int, default=600, help="seconds per bench.py run")
    ap.add_argument("--only", nargs="*", default=None, help="candidates instead of the built-in list")
    ap.add_argument("--no_combined", action="store_true", help="skip the run with every environment candidate at once")
    ap.add_argument("--bench_args", nargs=argparse.REMAINDER, default=[], help="passed to every bench.py run (last option)")
    ap.add_argument("--json_out", default="")
    a = ap.parse_args(argv)
    cands = a.only if a.only is not None else list(DEFAULT_CANDIDATES)
    rows = [run_one("default", {}, [], a, 29400, runner)]
    print(table(rows), flush=True)
    combined = {}
    for i, c in enumerate(cands):
        env, flags = split_candidate(c)
        rows.append(run_one(c, env, flags, a, 29401 + i, runner))
        if rows[-1]["ok"] and not flags:
            combined.update(env)
        print(table(rows[-1:]).splitlines()[-1], flush=True)
    if len(combined) > 1 and not a.no_combined:
        rows.append(run_one("all of the above that ran", combined, [], a, 29480, runner))
    print("\n" + table(rows), flush=True)
    if a.json_out:
        with open(a.json_out, "w") as f:
            json.dump(rows, f, indent=1)
    return 0 if rows[0]["ok"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
