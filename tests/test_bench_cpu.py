"""Host-side pieces of bench.py that need no GPU: the clock record, the workload description shared by both arms."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _FakeProc:
    def __init__(self, text):
        self.text = text

    def terminate(self):
        pass

    def communicate(self, timeout=None):
        return self.text, ""


def test_clock_record_takes_the_samples_under_load(bench):
    """Idle gaps between timed regions show the maximum clock at low power; the record must be the clock under load."""
    lines = []
    for _ in range(6):
        lines.append("0, 1965, 1965, 210.5, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active")
    for mhz in (1410, 1395, 1425):
        lines.append(f"0, {mhz}, 1965, 995.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active")
    s = bench.ClockSampler(0)
    s.proc = _FakeProc("\n".join(lines) + "\n")
    rec = s.stop()
    assert rec["sm_mhz"] == 1410 and rec["sm_max_mhz"] == 1965
    assert rec["reasons"] == ["sw_power_cap"]
    assert rec["samples"] == 9 and rec["samples_under_load"] == 3 and rec["power_w_max"] == 995.0


def test_clock_record_flags_thermal_slowdown(bench):
    s = bench.ClockSampler(0)
    s.proc = _FakeProc("0, 1200, 1965, 700.0, 0x40, Active, Active, Not Active, Not Active\n")
    rec = s.stop()
    assert "hw_slowdown" in rec["reasons"] and "hw_thermal_slowdown" in rec["reasons"]


def test_clock_record_without_nvidia_smi(bench):
    s = bench.ClockSampler(0)
    assert s.stop()["reasons"] == ["unavailable"]
    s.proc = _FakeProc("")
    assert s.stop()["reasons"] == ["no samples"]


def test_both_arms_describe_the_same_workload(bench):
    one = bench.workload_config(1)
    assert one["workload"] == "fp8_e4m3_gemm_8192x8192x8192" and (one["m"], one["n"], one["k"]) == (8192, 8192, 8192)
    for world in (2, 4, 8):
        cfg = bench.workload_config(world)
        assert cfg["parallelism"] == f"tp{world}" and cfg["hidden"] == 8192 and cfg["intermediate"] == 28672 and cfg["m"] == 2048
        assert "model" not in cfg
