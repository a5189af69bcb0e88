"""Host-side pieces of bench.py that need no GPU: the clock summary from NVML-style samples and from
nvidia-smi CSV lines, the reference arm's JSON line, and the workload arithmetic."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def _bench():
    sys.path.insert(0, str(ROOT))
    import bench
    return bench


def test_clock_summary_from_nvml_samples():
    bench = _bench()
    sampler = bench.ClockSampler(0)
    sampler.samples = [(1965, 1965, 0), (1700, 1965, 0x4), (1650, 1965, 0x4), (1965, 1965, 0)]
    summary = sampler.summary()
    assert summary["samples"] == 4 and summary["sm_max_mhz"] == 1965 and summary["sm_min_mhz"] == 1650
    assert summary["sm_mhz"] == (1700 + 1965) / 2
    assert summary["reasons"] == ["sw_power_cap"] and summary["source"] == "nvml"
    sampler.samples = [(1200, 1965, 0x8 | 0x40 | 0x20)]
    assert sampler.summary()["reasons"] == ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"]


def test_clock_summary_from_nvidia_smi_lines():
    bench = _bench()
    sampler = bench.ClockSampler(0)
    sampler.lines = ["0, 1965, 1965, 612.3, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
                     "0, 1830, 1965, 998.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
                     "garbage"]
    summary = sampler.summary()
    assert summary["samples"] == 2 and summary["reasons"] == ["sw_power_cap"] and summary["sm_max_mhz"] == 1965
    assert bench.ClockSampler(0).summary() == dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)


def test_workload_arithmetic():
    bench = _bench()
    assert len(bench.MODES) * len(bench.SHAPES) * len(bench.TOKENS) == 30
    assert bench.logical_ops((1536,)) == 2 * sum(2 * 1536 * n * k for k, n in bench.SHAPES)
    assert 1.0 < bench.TRAFFIC_OVER_ALGORITHMIC < 1.2
    assert bench.peaks()["bf16_tflops"] > 1000 and bench.peaks()["hbm_gbs"] > 6000


def test_reference_arm_prints_the_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0"],
                         capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "sparse_w8a8_linear_tops" and line["unit"] == "TOPS"
    assert line["value"] > 0 and line["e2e"] == {"value": line["value"], "unit": "TOPS", "h2d_bytes_per_step": 0,
                                                 "d2h_bytes_per_step": 0}
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["config"]["workload"] == "flux_sweep" and line["higher_is_better"] is True
