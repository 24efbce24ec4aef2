"""Command-line planner: tokens, FLOPs, memory per GPU, largest frame count and step time of a Wan preset at a
resolution and parallel layout, from the estimators of ``utils.flops`` (calibrated on measured B200 runs)."""
from __future__ import annotations

import torch


def main(argv=None) -> int:
    """``python -m teletron_b200.utils.plan --model wan2.1-14b-i2v --height 720 --width 1280 --frames 81 --gpus 8
    --cp 8``: print the plan for a Wan preset."""
    import argparse

    from ..models.wan import WanModel, wan_config
    from .flops import plan

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--model", default="wan2.1-1.3b-t2v")
    ap.add_argument("--height", type=int, default=480)
    ap.add_argument("--width", type=int, default=832)
    ap.add_argument("--frames", type=int, default=81)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--cp", type=int, default=1)
    ap.add_argument("--no-recompute", action="store_true")
    ap.add_argument("--tflops", type=float, default=850.0)
    a = ap.parse_args(argv)
    cfg = wan_config(a.model)
    with torch.device("meta"):
        n = sum(p.numel() for p in WanModel(cfg).parameters())
    r = plan(cfg, n, a.height, a.width, a.frames, a.gpus, a.cp, not a.no_recompute, tflops_per_gpu=a.tflops)
    print(f"{a.model}: {n / 1e9:.2f} B parameters, {r['tokens']:,} tokens per sample, {r['flops_per_sample']:.3e} FLOP per "
          f"sample ({'full' if not a.no_recompute else 'no'} recompute)")
    print(f"per GPU ({a.gpus} GPUs, CP {a.cp}): static {r['static_gib']:.1f} GiB + activations {r['activation_gib']:.1f} GiB "
          f"-> {'fits' if r['fits'] else 'does NOT fit'} in 179 GiB; largest frame count that fits: {r['max_frames']}")
    print(f"about {r['seconds_per_sample']:.2f} s per sample and CP group at {a.tflops:.0f} TFLOP/s per GPU")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
