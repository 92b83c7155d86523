"""Clock sampler against a stand-in NVML module (no GPU, no driver): only reads are issued."""
import time

from tinyinfinitrain_b200.utils.clocks import ClockSampler


class FakeNvml:
    NVML_CLOCK_SM = 1

    def __init__(self, masks):
        self.masks, self.calls, self.writes = list(masks), 0, 0

    def nvmlInit(self):
        pass

    def nvmlDeviceGetHandleByIndex(self, i):
        return ("h", i)

    def nvmlDeviceGetHandleByUUID(self, u):
        return ("h", u)

    def nvmlDeviceGetMaxClockInfo(self, h, kind):
        return 1965

    def nvmlDeviceGetClockInfo(self, h, kind):
        self.calls += 1
        return 1500 + 10 * (self.calls % 3)

    def nvmlDeviceGetCurrentClocksEventReasons(self, h):
        return self.masks[min(self.calls, len(self.masks) - 1)]


def test_sampler_collects_only_inside_the_window():
    fake = FakeNvml([0x4])
    s = ClockSampler(0, period_s=0.002, nvml=fake)
    s.launch()
    time.sleep(0.02)              # before begin(): nothing is recorded
    assert s._samples == []
    s.begin()
    time.sleep(0.05)
    s.end()
    n_at_end = len(s._samples)
    time.sleep(0.02)
    r = s.result()
    assert r["backend"] == "nvml" and r["samples"] >= 5 and r["samples"] <= n_at_end + 1
    assert r["sm_max_mhz"] == 1965 and 1500 <= r["sm_mhz"] <= 1520
    assert r["reasons"] == ["sw_power_cap"]


def test_sampler_reports_thermal_reasons_and_uuid_lookup():
    fake = FakeNvml([0x0, 0x40 | 0x20, 0x8])
    s = ClockSampler(3, uuid="01234567-89ab-cdef-0123-456789abcdef", period_s=0.001, nvml=fake)
    s.launch()
    assert s._handle == ("h", "GPU-01234567-89ab-cdef-0123-456789abcdef")
    s.begin()
    time.sleep(0.03)
    s.end()
    r = s.result()
    assert "hw_slowdown" in r["reasons"]


def test_sampler_without_driver_returns_empty_record():
    class Broken(FakeNvml):
        def nvmlInit(self):
            raise RuntimeError("no driver")

    s = ClockSampler(0, nvml=Broken([0]))
    s.launch()  # falls back to nvidia-smi, which may be absent too
    s.begin()
    s.end()
    r = s.result()
    assert r["samples"] == 0 and r["sm_mhz"] is None
