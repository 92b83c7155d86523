"""Failure detection between ranks, on the host.

The reference has none: errors are CHECK/LOG(FATAL) aborts (infini_train/src/device.cc:12,
dispatcher.h:41).  A multi-GPU job needs the surviving ranks to find out, *before their next
launch*, that a peer is gone -- otherwise their next collective or fused kernel waits for a peer
that will never arrive.  Three layers:

* ``HealthMonitor``: every rank publishes ``ok:<step>`` (or ``failed:<reason>``) under its own key
  of the job's c10d store after each step; ``check()`` reads the peers' keys and raises
  ``PeerFailure`` if one reported a failure or has not reached the expected step within the
  timeout.  ``guard()`` publishes the failure when the rank's own step raises.
* a short process-group timeout (``init_process_group(timeout=...)``) turns a collective a dead
  peer never joins into an error instead of a hang;
* on the device every wait on a peer's flag is bounded and records ``kStatusPeerTimeout`` in the
  library status word (``_lib.C.status_read``), which ``check_device_status`` turns into an exception.

Recovery is restart from the last checkpoint (``utils.checkpoint``); there is no in-job elasticity.
"""
from __future__ import annotations

import contextlib
import time
from typing import Optional

import torch.distributed as dist


class PeerFailure(RuntimeError):
    def __init__(self, rank: int, reason: str):
        super().__init__(f"rank {rank} failed: {reason}")
        self.rank, self.reason = rank, reason


class HealthMonitor:
    def __init__(self, store=None, rank: Optional[int] = None, world: Optional[int] = None, prefix: str = "titb_health"):
        if store is None:
            from torch.distributed.distributed_c10d import _get_default_store

            store = _get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix = prefix

    def _key(self, r: int) -> str:
        return f"{self.prefix}/{r}"

    def beat(self, step: int) -> None:
        self.store.set(self._key(self.rank), f"ok:{step}")

    def fail(self, reason: str) -> None:
        self.store.set(self._key(self.rank), f"failed:{reason}")

    def check(self, step: int, timeout_s: float = 5.0, poll_s: float = 0.02) -> None:
        """Raises PeerFailure unless every peer has published ``ok:<s>`` with s >= step."""
        deadline = time.monotonic() + timeout_s
        for r in range(self.world):
            if r == self.rank:
                continue
            while True:
                val = None
                if self.store.check([self._key(r)]):
                    val = self.store.get(self._key(r)).decode()
                if val is not None and val.startswith("failed:"):
                    raise PeerFailure(r, val[len("failed:"):])
                if val is not None and val.startswith("ok:") and int(val[3:]) >= step:
                    break
                if time.monotonic() > deadline:
                    raise PeerFailure(r, f"no heartbeat for step {step} within {timeout_s:.1f}s (last: {val})")
                time.sleep(poll_s)

    @contextlib.contextmanager
    def guard(self):
        """Publishes this rank's failure to the peers when the guarded block raises."""
        try:
            yield
        except BaseException as e:  # noqa: BLE001
            try:
                self.fail(f"{type(e).__name__}: {e}")
            finally:
                raise


def check_device_status(clear: bool = True) -> None:
    """Raises if a device-side bounded wait gave up since the last check."""
    from .._lib import C

    code = int(C.status_read(clear))
    if code == 1:
        raise RuntimeError("a tcgen05/TMA pipeline wait timed out inside a kernel (status 1)")
    if code == 2:
        raise PeerFailure(-1, "a device-side wait on another GPU's flag timed out (status 2)")
    if code != 0:
        raise RuntimeError(f"kernel status word = {code}")
