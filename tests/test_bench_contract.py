"""Driver-facing contract of the two root scripts, as far as it can be checked without a GPU."""
import importlib.util
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, name + ".py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_prints_one_unavailable_line_and_exits_zero():
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "8",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]


def test_clock_samples_are_summarised_under_load_only(tmp_path):
    bench = _load("bench")
    p = tmp_path / "clocks.csv"
    p.write_text(
        "0, 345, 1965, 150.0, 0x0, Not Active, Not Active, Not Active, Not Active\n"      # idle sample
        "0, 1800, 1965, 950.0, 0x4, Not Active, Not Active, Not Active, Active\n"
        "0, 1700, 1965, 990.0, 0x4, Not Active, Not Active, Not Active, Active\n"
        "0, 1750, 1965, 970.0, 0x4, Not Active, Not Active, Not Active, Active\n"
        "1, 1000, 1965, 900.0, 0x8, Not Active, Active, Not Active, Not Active\n"         # a GPU outside the run
        "garbage line\n")
    c = bench._parse_clocks(str(p), 1)
    assert c["sm_mhz"] == 1750 and c["sm_max_mhz"] == 1965 and c["reasons"] == ["sw_power_cap"]
    assert c["samples"] == 4 and c["power_w_max"] == 990.0
    assert bench._parse_clocks(str(tmp_path / "missing.csv"), 1)["samples"] == 0


def test_entry_points_exist():
    entry = _load("__graft_entry__")
    assert callable(entry.build) and callable(entry.smoke)
