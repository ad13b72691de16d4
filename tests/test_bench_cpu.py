"""bench.py's host logic without a GPU: the clock sampler against a fake NVML, and the reference arm's JSON line on
the smallest workload (the reference's own CPU build, or the CPU restatement where that library is not built)."""
import importlib.util
import json
import subprocess
import sys
import time
import types
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def fake_nvml(clock_of_call, mask_of_call):
    m = types.ModuleType("pynvml")
    m.NVML_CLOCK_SM = 1
    m.nvmlClocksEventReasonHwSlowdown, m.nvmlClocksEventReasonHwThermalSlowdown = 0x8, 0x40
    m.nvmlClocksEventReasonSwThermalSlowdown, m.nvmlClocksEventReasonSwPowerCap = 0x20, 0x4
    m.calls = {"n": 0, "set": 0}
    m.nvmlInit = lambda: None
    m.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)

    def by_uuid(u):
        raise RuntimeError("no such device")  # as when the CUDA runtime is absent: the sampler falls back to the index
    m.nvmlDeviceGetHandleByUUID = by_uuid

    def clock(h, kind):
        m.calls["n"] += 1
        return clock_of_call(m.calls["n"])
    m.nvmlDeviceGetClockInfo = clock
    m.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965
    m.nvmlDeviceGetCurrentClocksEventReasons = lambda h: mask_of_call(m.calls["n"])
    return m


def test_clock_sampler_reads_and_never_sets(monkeypatch):
    bench = load_bench()
    nv = fake_nvml(lambda n: 1500 if n <= 2 else 1900, lambda n: 0x4 if n > 2 else 0x8)
    monkeypatch.setitem(sys.modules, "pynvml", nv)
    s = bench.ClockSampler(0)
    s.start()
    s.wait_started()
    while len(s.samples) < 2:  # the warm-up's samples: a slow clock and a hardware slowdown that must not be counted
        time.sleep(0.01)
    s.mark()
    first = len(s.samples)
    while len(s.samples) < first + 3:
        time.sleep(0.01)
    out = s.stop()
    assert out["sm_mhz"] == 1900.0 and out["sm_max_mhz"] == 1965.0
    assert out["reasons"] == ["sw_power_cap"], "only what was active inside the timed region, by the recipe's names"
    assert out["samples"] >= 3 and "NVML" in out["source"]
    assert not [n for n in dir(nv) if "Set" in n or "Reset" in n], "the fake offers nothing that sets, and none was missed"


def test_clock_sampler_without_nvml_says_so(monkeypatch):
    bench = load_bench()
    broken = types.ModuleType("pynvml")

    def init():
        raise RuntimeError("driver not loaded")
    broken.nvmlInit = init
    monkeypatch.setitem(sys.modules, "pynvml", broken)
    s = bench.ClockSampler(0)
    s.start()
    s.wait_started(limit=0.2)
    out = s.stop()
    assert out["sm_mhz"] is None and out["reasons"] == ["NVML unavailable"]


def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                        "--workload", "diamond64"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, "one JSON line on stdout"
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "atom_evals_per_s" and d["unit"] == "atom-evals/s"
    assert d["n_gpus"] == 1 and d["steps"] == 1 and d["warmup"] == 0 and d["higher_is_better"] is True
    assert d["value"] > 0 and abs(d["value"] - 64 / (d["ms_per_step"] * 1e-3)) <= 1e-6 * d["value"]
    assert d["config"]["workload"] == "diamond64" and "model" in d["config"]
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    assert d["e2e"] == {"value": d["value"], "unit": d["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["vs_baseline"] is None
