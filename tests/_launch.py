"""Child-job launcher for the multi-rank tests: the job runs in a process group of its own, and when it does not end
within the limit the whole group (torchrun and every worker it started) is terminated -- by the group id this
function created, never by a name pattern -- so no orphaned worker keeps a GPU."""
import os
import signal
import subprocess
from types import SimpleNamespace


def run_group(cmd, env=None, timeout=600, cwd=None):
    p = subprocess.Popen(cmd, env=env, cwd=cwd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True,
                         start_new_session=True)
    try:
        out, err = p.communicate(timeout=timeout)
        return SimpleNamespace(returncode=p.returncode, stdout=out, stderr=err)
    except subprocess.TimeoutExpired:
        for sig, grace in ((signal.SIGTERM, 15), (signal.SIGKILL, 15)):
            try:
                os.killpg(p.pid, sig)          # the session leader's pid is the group id
            except ProcessLookupError:
                break
            try:
                out, err = p.communicate(timeout=grace)
                break
            except subprocess.TimeoutExpired:
                continue
        else:
            out, err = "", ""
        return SimpleNamespace(returncode=-9, stdout=out or "", stderr=(err or "") + f"\n[no result within {timeout} s: process group terminated]")
