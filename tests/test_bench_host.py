"""Host-side pieces of bench.py that need no GPU: the clock sampler against a fake NVML."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


class FakeNvml:
    NVML_CLOCK_SM = 1

    def __init__(self, clocks, reasons):
        self.clocks, self.reasons, self.i = clocks, reasons, 0

    def nvmlDeviceGetHandleByIndex(self, index):
        return ("handle", index)

    def nvmlDeviceGetMaxClockInfo(self, h, which):
        return 1965

    def nvmlDeviceGetClockInfo(self, h, which):
        c = self.clocks[min(self.i, len(self.clocks) - 1)]
        return c

    def nvmlDeviceGetPowerUsage(self, h):
        return 900000 + self.i

    def nvmlDeviceGetCurrentClocksEventReasons(self, h):
        r = self.reasons[min(self.i, len(self.reasons) - 1)]
        self.i += 1
        return r


def test_clock_sampler_samples_only_while_work_is_in_flight():
    import bench
    nv = FakeNvml([1400, 1350, 1300, 1965], [0x4, 0x4, 0x0, 0x0])
    cs = bench.ClockSampler(0, nvml=nv)
    polls = {"n": 0}

    def done():
        polls["n"] += 1
        return polls["n"] > 3           # three samples under load, then the end event has completed

    cs.poll_until(done)
    out = cs.summary()
    assert out["samples"] == 3 and out["sm_mhz"] == 1350.0 and out["sm_min_mhz"] == 1300.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"]
    assert cs.idle_sample[0] == 1965.0   # taken after the region, not part of the statistics


def test_clock_sampler_short_region_falls_back_to_one_sample_after():
    import bench
    cs = bench.ClockSampler(0, nvml=FakeNvml([1965], [0]))
    cs.poll_until(lambda: True)
    out = cs.summary()
    assert out["samples"] == 0 and out["sm_mhz"] == 1965.0 and "after" in out["when"]


def test_clock_sampler_without_nvml_is_inert():
    import bench

    class Broken:
        def nvmlDeviceGetHandleByIndex(self, i):
            raise RuntimeError("no NVML")

    cs = bench.ClockSampler(0, nvml=Broken())
    cs.poll_until(lambda: False, limit_s=0.01)
    assert cs.summary()["samples"] == 0
