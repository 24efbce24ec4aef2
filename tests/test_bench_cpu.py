"""The host-side pieces of bench.py that need no GPU: token arithmetic, the clock-sample summary that goes into the
JSON line, and the reference arm's answer when the reference cannot run."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _Proc:
    def terminate(self):
        pass

    def wait(self, timeout=None):
        return 0


def test_token_arithmetic_and_headline_constants():
    b = _bench()
    assert b.tokens_per_sample(81, 480, 832) == b.TOKENS_PER_SAMPLE == 32_760
    assert b.tokens_per_sample(81, 720, 1280) == 75_600 and b.tokens_per_sample(161, 720, 1280) == 147_600
    assert b.METRIC == "wan2.1_1.3b_t2v_480p81f_train_tokens_per_s" and b.GLOBAL_BATCH == 8


def test_clock_samples_are_summarised_for_the_right_gpu(tmp_path, monkeypatch):
    b = _bench()
    monkeypatch.setenv("TT_BENCH_LOG_DIR", str(tmp_path / "logs"))
    assert b.clock_log_dir() == str(tmp_path / "logs") and (tmp_path / "logs").is_dir()
    rows = [
        "0, 210, 1965, 140.1, 0x0000000000000001, Not Active, Not Active, Not Active, Not Active",     # idle sample
        "0, 1700, 1965, 990.2, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "1, 1200, 1965, 500.0, 0x0000000000000004, Active, Not Active, Not Active, Active",            # another GPU
        "0, 1650, 1965, 995.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "0, 1680, 1965, 999.9, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
        "garbage line",
    ]
    path = tmp_path / "clocks.csv"
    path.write_text("\n".join(rows) + "\n")
    out = b.clock_sampler_stop(_Proc(), open(path), str(path), device_index=0)
    assert out == {"sm_mhz": 1680.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 4}
    other = b.clock_sampler_stop(_Proc(), open(path), str(path), device_index=1)
    assert other["reasons"] == ["hw_slowdown", "sw_power_cap"] and other["sm_mhz"] == 1200.0
    assert b.clock_sampler_stop(None, None, str(path)) == {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}


def test_reference_arm_answers_on_a_box_without_a_gpu():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-500:]
    line = [l for l in r.stdout.splitlines() if l.startswith("{")][-1]
    msg = json.loads(line)
    assert msg["impl"] == "reference" and "unavailable" in msg and isinstance(msg["unavailable"], str)
