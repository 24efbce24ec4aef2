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


def _ref_args(b, extra=()):
    import argparse

    ns = argparse.Namespace(gpus=1, steps=2, warmup=3, impl="reference", model="wan2.1-1.3b-t2v", cp=1, recompute=False,
                            layers=0, frames=9, height=64, width=64, global_batch=2, init_on_device=False,
                            ref_no_recompute=False, ref_recompute_only=False, fused_comm="auto")
    for k, v in extra:
        setattr(ns, k, v)
    return ns


def test_reference_arm_prints_a_full_line_when_driven_on_cpu(capsys):
    """The whole reference arm (both activation settings probed, device-timed pass, end-to-end pass, result line)
    runs on CPU with a tiny shape of the reference's own model file, so that a broken result line cannot ship."""
    from conftest import reference_file

    b = _bench()
    wan = reference_file("teletron/models/wan/wan_model.py")
    if wan is None:
        import pytest
        pytest.skip("reference tree not available")
    shape = {"dims": (128, 4, 2, 512), "text_dim": 64, "text_len": 32, "freq_dim": 64}
    rc = b.run_reference(_ref_args(b), device="cpu", shape=shape, ref_root=wan.parents[3])
    assert rc == 0
    line = [l for l in capsys.readouterr().out.splitlines() if l.startswith("{")][-1]
    msg = json.loads(line)
    assert msg["impl"] == "reference" and "unavailable" not in msg
    tok = b.tokens_per_sample(9, 64, 64)
    assert msg["config"]["seq_len"] == tok == 48 and msg["config"]["global_batch"] == 2
    assert msg["steps"] == 2 and msg["warmup"] == 3 and msg["value"] > 0 and msg["ms_per_step"] > 0
    assert abs(msg["value"] - 2 * tok / (msg["ms_per_step"] * 1e-3)) < 1e-6 * msg["value"]
    e = msg["e2e"]
    assert e["value"] > 0 and e["steps"] == 2 and e["d2h_bytes_per_step"] == 4
    assert e["h2d_bytes_per_step"] == 2 * 4 * (16 * 3 * 8 * 8 + 32 * 64)      # fp32 on CPU: latents + context, 2 samples
    assert set(msg["config"]["recompute_settings_tried"]) == {"none", "per-block checkpointing (the reference's shipped setting)"}
    assert msg["config"]["recompute"] in msg["config"]["recompute_settings_tried"]
    assert msg["metric"].endswith("_64p9f_train_tokens_per_s") and msg["vs_baseline"] is None
    assert isinstance(e["last_loss"], float)


def test_reference_result_line_names_the_headline_metric():
    b = _bench()
    a = _ref_args(b, (("frames", 81), ("height", 480), ("width", 832), ("global_batch", 8), ("steps", 20), ("warmup", 5)))
    r = b.reference_result(a, tok_sample=32760, gbs=8, desc="d", ms_dev=20 * 24_000.0, ms_e2e=10 * 24_100.0, e2e_steps=10,
                           h2d_bytes_per_step=1, clocks={}, last_loss=1.0, recompute="none", settings_tried={})
    assert r["metric"] == b.METRIC and abs(r["value"] - 8 * 32760 / 24.0) < 1e-6
    assert abs(r["e2e"]["value"] - 8 * 32760 / 24.1) < 1e-6 and r["e2e"]["steps"] == 10
    assert abs(r["vs_baseline"] - r["value"] / 1090.0) < 1e-9
