"""The reference arm of bench.py runs on host cores only and must print the contract's line."""

from __future__ import annotations

import json
import pathlib
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_contract_line():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0", "--workload", "c1", "--cpu-tokens", "2000"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "GB/s" and d["higher_is_better"] is True
    assert d["metric"] == "decode_attn_hbm_gbs" and d["value"] > 0 and d["steps"] == 1
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"] == d["e2e"]["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    assert "workload" in d["config"]


def _bench_module():
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_clock_summary_reads_the_loaded_samples_and_the_reasons():
    bench = _bench_module()
    s = bench.ClockSampler(0, enabled=False)
    s.lines = ["210, 1965, Not Active, Not Active, Not Active, Not Active",      # idle before the region
               "1965, 1965, Not Active, Not Active, Not Active, Not Active",
               "1830, 1965, Not Active, Not Active, Not Active, Active",
               "1845, 1965, Not Active, Not Active, Not Active, Active",
               "garbage line",
               "[N/A], 1965, Not Active, Not Active, Not Active, Not Active"]
    got = s.summary()
    assert got["sm_max_mhz"] == 1965.0 and got["samples"] == 4
    assert got["reasons"] == ["sw_power_cap"]
    assert got["sm_mhz"] in (1845.0, 1905.0)  # the median of the upper half: the idle sample does not count
    empty = bench.ClockSampler(0, enabled=False).summary()
    assert empty["sm_mhz"] is None and empty["reasons"] == []


def test_both_arms_print_the_same_config_for_the_same_batch():
    bench = _bench_module()
    a = bench._config("c2", 0, 64, 1442787328.0)
    b = bench._config("c2", 0, 64, 1442787328)
    assert a == b and set(a) == {"workload", "seed", "batch", "kv_bytes_job"}
    assert a["workload"].startswith("c2: ")
