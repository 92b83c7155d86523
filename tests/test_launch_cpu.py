"""The child-job launcher of the multi-rank tests: normal completion, and a job that outlives its limit together
with a grandchild it started (both must be gone afterwards)."""
import os
import sys
import time

from _launch import run_group


def test_normal_completion():
    r = run_group([sys.executable, "-c", "import sys; print('hi'); sys.exit(3)"], timeout=60)
    assert r.returncode == 3 and r.stdout.strip() == "hi"


def test_timeout_ends_the_whole_group(tmp_path):
    marker = tmp_path / "pids"
    code = ("import os, subprocess, sys, time\n"
            f"c = subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(600)'])\n"
            f"open({str(marker)!r}, 'w').write(f'{{os.getpid()}} {{c.pid}}')\n"
            "time.sleep(600)\n")
    t0 = time.time()
    r = run_group([sys.executable, "-c", code], timeout=3)
    assert r.returncode == -9 and "process group terminated" in r.stderr and time.time() - t0 < 40
    parent, child = (int(x) for x in open(marker).read().split())
    time.sleep(0.5)
    for pid in (parent, child):
        try:
            os.kill(pid, 0)
            alive = open(f"/proc/{pid}/stat").read().split()[2] != "Z"     # a zombie awaiting its reaper is gone for our purposes
        except (ProcessLookupError, FileNotFoundError):
            alive = False
        assert not alive, pid
