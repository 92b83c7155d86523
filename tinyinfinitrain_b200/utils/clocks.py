"""Read-only sampling of a GPU's SM clock and clock-event ("throttle") reasons while a timed region runs.

Two back ends, both of which only *read* state:

* NVML through ``pynvml`` in a thread of this process (preferred: the first sample is taken within a
  few milliseconds, which matters for timed regions of a few hundred milliseconds);
* an ``nvidia-smi --query-gpu ... -lms`` child process whose time-stamped lines are filtered to the
  window between :meth:`ClockSampler.begin` and :meth:`ClockSampler.end` (it needs a second or more to
  start on a node with many GPUs, so it is started early with :meth:`ClockSampler.launch`).

Nothing here sets clocks, power limits or any other device state.
"""
from __future__ import annotations

import datetime as _dt
import os
import statistics
import subprocess
import threading
import time
from typing import Dict, List, Optional

# NVML clock-event reason bits (nvml.h: nvmlClocksEventReason*)
_REASON_BITS = {
    "sw_power_cap": 0x0000000000000004,
    "hw_slowdown": 0x0000000000000008,
    "sw_thermal_slowdown": 0x0000000000000020,
    "hw_thermal_slowdown": 0x0000000000000040,
}
_SMI_QUERY = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
_SMI_REASONS = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]


class ClockSampler:
    def __init__(self, index: int = 0, uuid: Optional[str] = None, period_s: float = 0.01, nvml=None):
        """``index`` / ``uuid`` name the GPU (the UUID wins when NVML is used: CUDA and NVML may order
        devices differently).  ``nvml`` lets a test pass a stand-in for the ``pynvml`` module."""
        self.index, self.uuid, self.period = index, uuid, period_s
        self._nvml, self._handle = nvml, None
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._active = threading.Event()
        self._samples: List[Dict] = []
        self._smi = None
        self._smi_path = f"/tmp/titb_clocks_{os.getpid()}.csv"
        self._t_begin = self._t_end = None
        self.backend = "none"

    # ---- life cycle: launch() early, begin()/end() around the timed region, result() after ---------
    def launch(self) -> None:
        if self._open_nvml():
            self.backend = "nvml"
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
            return
        try:
            self._smi_file = open(self._smi_path, "w")
            self._smi = subprocess.Popen(["nvidia-smi", f"--query-gpu={_SMI_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=self._smi_file,
                                         stderr=subprocess.DEVNULL)
            self.backend = "nvidia-smi"
        except Exception:  # noqa: BLE001 - no nvidia-smi on this machine
            self._smi = None

    def begin(self) -> None:
        self._t_begin = time.time()
        self._active.set()

    def end(self) -> None:
        self._t_end = time.time()
        self._active.clear()

    def result(self) -> Dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "backend": self.backend}
        samples = self._samples
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
        if self._smi is not None:
            self._smi.terminate()
            try:
                self._smi.wait(timeout=5)
            except Exception:  # noqa: BLE001
                self._smi.kill()
            self._smi_file.close()
            samples = self._parse_smi()
            try:
                os.remove(self._smi_path)
            except OSError:
                pass
        if samples:
            reasons = set()
            for s in samples:
                reasons.update(s["reasons"])
            out.update(sm_mhz=statistics.median(s["sm"] for s in samples), sm_max_mhz=max(s["max"] for s in samples),
                       reasons=sorted(reasons), samples=len(samples))
        return out

    # ---- NVML -----------------------------------------------------------------------------------
    def _open_nvml(self) -> bool:
        try:
            if self._nvml is None:
                import pynvml

                self._nvml = pynvml
            n = self._nvml
            n.nvmlInit()
            self._handle = None
            if self.uuid:
                u = self.uuid if str(self.uuid).startswith("GPU-") else f"GPU-{self.uuid}"
                try:
                    try:
                        self._handle = n.nvmlDeviceGetHandleByUUID(u)
                    except TypeError:  # bindings that want bytes
                        self._handle = n.nvmlDeviceGetHandleByUUID(u.encode())
                except Exception:  # noqa: BLE001 - a UUID string NVML does not accept: fall back to the index
                    self._handle = None
            if self._handle is None:
                self._handle = n.nvmlDeviceGetHandleByIndex(self.index)
            self._max = int(n.nvmlDeviceGetMaxClockInfo(self._handle, n.NVML_CLOCK_SM))
            self._read_nvml()  # fail here rather than in the thread
            return True
        except Exception:  # noqa: BLE001 - no driver / no pynvml: fall back to nvidia-smi
            self._handle = None
            return False

    def _read_nvml(self) -> Dict:
        n = self._nvml
        sm = int(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
        get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        mask = int(get(self._handle))
        return {"sm": sm, "max": self._max, "reasons": [k for k, b in _REASON_BITS.items() if mask & b]}

    def _loop(self) -> None:
        while not self._stop.is_set():
            if self._active.is_set():
                try:
                    self._samples.append(self._read_nvml())
                except Exception:  # noqa: BLE001
                    pass
            self._stop.wait(self.period)

    # ---- nvidia-smi -------------------------------------------------------------------------------
    def _parse_smi(self) -> List[Dict]:
        out = []
        try:
            lines = open(self._smi_path).read().splitlines()
        except OSError:
            return out
        for line in lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = _dt.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                sm, mx = float(parts[1]), float(parts[2])
            except ValueError:
                continue
            if self._t_begin is not None and self._t_end is not None and not (self._t_begin - 0.05 <= ts <= self._t_end + 0.05):
                continue
            out.append({"sm": sm, "max": mx,
                        "reasons": [n for n, v in zip(_SMI_REASONS, parts[4:8]) if v.lower().startswith("active")]})
        return out
