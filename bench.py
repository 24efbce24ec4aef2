#!/usr/bin/env python
"""Headline benchmark: Wan2.1-1.3B t2v training throughput (tokens/s) at 480P x 81 frames.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched under torchrun)
    python bench.py --impl reference ...                     (the reference's own model code)

One step = one optimizer step over a global batch of 8 samples (32,760 tokens each), bf16,
synthetic latents / text embeddings, random-init weights, AdamW.  The same global batch is
used at every N (strong scaling): DP over the ranks that are not used for Ulysses CP, gradient
accumulation when fewer than 8 replicas exist.  At N > 1 every Ulysses size that divides N is
tried for a few steps (`layouts` in the JSON line) and the fastest layout is measured in full.
Rank 0 prints one JSON line.

Other rows of the same benchmark: ``--model wan2.1-14b-i2v --cp 8 --height 720 --width 1280 --global-batch 1
--recompute`` (any Wan preset, resolution, frame count, global batch, Ulysses size); the metric name then carries the
preset and resolution.  ``peak_mem_gib`` is the allocator's high-water mark, max over ranks.

`value` is timed on the device with CUDA events with inputs already resident; `e2e` repeats
the measurement through ``Trainer.train_step`` with every step's inputs copied from pinned host
memory and the loss read back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "wan2.1_1.3b_t2v_480p81f_train_tokens_per_s"
FRAMES, HEIGHT, WIDTH = 81, 480, 832
TOKENS_PER_SAMPLE = 21 * 30 * 52  # 32,760
GLOBAL_BATCH = 8
PUBLISHED_TOKENS_PER_S_PER_GPU = 1090.0  # 21.6 FPS/node on 16 x H800, read off ComparativeGraph.jpg
PUBLISHED_720P_TOKENS_PER_S_PER_GPU = 567.0  # 4.8 FPS/node at 720P x 81, same chart


def tokens_per_sample(frames: int, height: int, width: int) -> int:
    """Latent frames x (H/16) x (W/16): 8x VAE, 4x temporal compression, patch (1, 2, 2)."""
    return ((frames - 1) // 4 + 1) * (height // 16) * (width // 16)


def clock_log_dir() -> str:
    """Folder for the raw nvidia-smi samples (the JSON line carries their summary)."""
    d = os.environ.get("TT_BENCH_LOG_DIR") or os.path.join(tempfile.gettempdir(), "teletron_b200_bench")
    os.makedirs(d, exist_ok=True)
    return d


def clock_sampler_start(path: str):
    q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    try:
        f = open(path, "w")
        return subprocess.Popen(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                stdout=f, stderr=subprocess.DEVNULL), f
    except Exception:
        return None, None


def clock_sampler_stop(proc, f, path: str, device_index: int = 0):
    out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    if proc is None:
        return out
    proc.terminate()
    try:
        proc.wait(timeout=5)
    except Exception:
        proc.kill()
    f.close()
    sm, mx, reasons = [], [], set()
    try:
        for line in open(path):
            c = [x.strip() for x in line.split(",")]
            if len(c) < 9 or not c[0].isdigit() or int(c[0]) != device_index:
                continue
            try:
                sm.append(float(c[1]))
                mx.append(float(c[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), c[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
    except FileNotFoundError:
        return out
    if sm:
        busy = [s for s in sm if s > 0.5 * max(sm)] or sm
        out["sm_mhz"] = statistics.median(busy)
        out["sm_max_mhz"] = max(mx)
        out["reasons"] = sorted(reasons)
        out["samples"] = len(sm)
    return out


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


# ------------------------------------------------------------------------------ ours
def candidate_layouts(world: int, gbs: int, cp_flag: int, tp: int = 1):
    """Ulysses sizes to measure at `world` GPUs: the one asked for, or every power of two that divides the world and
    leaves a data-parallel size that divides the global batch; data parallelism only (cp = 1) comes last."""
    if cp_flag > 0:
        return [cp_flag]
    world //= tp
    out = [cp for cp in (8, 4, 2, 1) if cp <= world and world % cp == 0 and gbs % (world // cp) == 0]
    return out or [world]


def layout_name(world: int, cp: int, tp: int = 1) -> str:
    dp = world // (cp * tp)
    return f"dp{dp}" + (f"xtp{tp}" if tp > 1 else "") + (f"xcp{cp}" if cp > 1 else "")


def run_ours(a):
    import gc

    import torch
    import torch.distributed as dist

    from teletron_b200.data import SyntheticLatentDataset
    from teletron_b200.ops import _lib
    from teletron_b200.parallel import state as mpu
    from teletron_b200.train import Trainer, make_forward_step, parse_args
    from teletron_b200.train.hunyuan_step import make_hunyuan_forward_step

    rank, world, local = dist_env()
    assert world == a.gpus, f"WORLD_SIZE {world} != --gpus {a.gpus} (launch N > 1 under torchrun)"
    if not torch.cuda.is_available():
        raise SystemExit("bench.py measures on a GPU: no CUDA device on this machine")
    frames, height, width, gbs = a.frames, a.height, a.width, a.global_batch
    headline = (a.model == "wan2.1-1.3b-t2v" and (frames, height, width, gbs) == (FRAMES, HEIGHT, WIDTH, GLOBAL_BATCH))
    tok_sample = tokens_per_sample(frames, height, width)
    i2v = "i2v" in a.model
    hunyuan = a.model.startswith("hunyuan")
    tp = a.tp
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    fwd = make_hunyuan_forward_step() if hunyuan else make_forward_step()
    # the same global batch at every N and in every layout: sample i (latents, text, noise, timestep) is a function
    # of i alone, and data-parallel rank d takes samples [d * n_mb, (d + 1) * n_mb)
    if hunyuan:
        from teletron_b200.data.fake import SyntheticHunyuanDataset

        ds = SyntheticHunyuanDataset(frames, height, width, i2v=i2v, seed=1234)
    else:
        ds = SyntheticLatentDataset(frames, height, width, i2v=i2v, seed=1234, fixed_noise=True)

    def build(cp):
        argv = ["--model", "ParallelHunyuanVideoModel" if hunyuan else "ParallelWanModel", "--model-preset", a.model,
                "--tensor-model-parallel-size", str(tp), "--bf16", "--micro-batch-size", "1",
                "--global-batch-size", str(gbs), "--train-iters", "1000000", "--lr", "1e-5",
                "--weight-decay", "1e-2", "--clip-grad", "1.0", "--context-parallel-size", str(cp),
                "--num-frames", str(frames), "--video-resolution", str(height), str(width), "--synthetic-latents",
                "--log-interval", "1000000", "--seed", "1234"]
        if i2v:
            argv += ["--task-type", "i2v"]
        if a.init_on_device or "14b" in a.model or "13b" in a.model:
            argv.append("--init-on-device")
        if world > 1:
            argv.append("--use-distributed-optimizer")
        argv += ["--fused-comm", a.fused_comm]
        if a.no_overlap:
            argv.append("--no-overlap-grad-reduce")
        if a.recompute:
            argv += ["--recompute-granularity", "full", "--recompute-method", "block", "--recompute-num-layers", "1000"]
        if a.layers:
            argv += ["--num-layers", str(a.layers)]
        targs = parse_args(argv=argv)
        tr = Trainer(targs, build_data=False)
        n_mb = targs.num_micro_batches
        d = mpu.get_data_parallel_rank() if world > 1 else 0
        host = []
        for i in range(d * n_mb, (d + 1) * n_mb):
            host.append({k: v.unsqueeze(0).pin_memory() for k, v in ds[i].items()})
        dev_pool = [{k: v.to(tr.device) for k, v in b.items()} for b in host]
        return tr, host, dev_pool

    def teardown(tr):
        cpx = getattr(getattr(tr.model, "module", tr.model), "cp", None)
        if cpx is not None:
            cpx.fused = None
        tr.model = tr.optimizer = tr.buffer = tr.arena = None
        mpu.destroy_model_parallel()
        gc.collect()
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

    def cycle(pool):
        i = 0
        while True:
            yield pool[i % len(pool)]
            i += 1

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(tr, pool, steps, read_loss):
        it = cycle(pool)
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.launch_count()
        e0.record()
        last = None
        for _ in range(steps):
            loss_dict, _, _, _ = tr.train_step(fwd, it)
            if read_loss:
                last = float(loss_dict["loss"])  # device -> host read of the step's result
        e1.record()
        sync_all()
        ms = e0.elapsed_time(e1)
        t = torch.tensor([ms], dtype=torch.float64, device=tr.device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()), _lib.launch_count() - l0, last

    def warm(tr, pool, n):
        """n untimed steps; returns the loss of the first one (the parity value: same weights, same batch)."""
        first = None
        for i in range(n):
            ld, _, _, _ = tr.train_step(fwd, cycle(pool))
            if i == 0:
                first = float(ld["loss"])
        sync_all()
        _lib.check_status()
        return first

    cands = candidate_layouts(world, gbs, a.cp, tp)
    layouts = {}
    tr = host = dev_pool = None
    built = None
    trial_steps, trial_warm = 3, 3
    for i, cp in enumerate(cands):
        name = layout_name(world, cp, tp)
        try:
            tr, host, dev_pool = build(cp)
            built = cp
            if len(cands) == 1:
                break
            first = warm(tr, dev_pool, trial_warm)
            ms, _, _ = timed(tr, dev_pool, trial_steps, read_loss=False)
            layouts[name] = {"tokens_per_s": gbs * tok_sample * trial_steps / (ms * 1e-3), "ms_per_step": ms / trial_steps,
                             "steps": trial_steps, "warmup": trial_warm, "loss_first_step": first,
                             "fused_ulysses": bool(getattr(getattr(getattr(tr.model, "module", tr.model), "cp", None),
                                                           "fused", None))}
        except Exception as e:  # a layout that cannot run (memory, unsupported split) is reported, not fatal
            if len(cands) == 1:
                raise
            layouts[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
            built = None
        if i < len(cands) - 1 and tr is not None:
            teardown(tr)
            tr = host = dev_pool = None
    ok = {k: v for k, v in layouts.items() if "tokens_per_s" in v}
    if len(cands) > 1:
        if not ok:
            raise SystemExit(f"no layout ran: {layouts}")
        best = max(ok, key=lambda k: ok[k]["tokens_per_s"])
        best_cp = next(c for c in cands if layout_name(world, c, tp) == best)
        if built != best_cp:
            if tr is not None:
                teardown(tr)
            tr, host, dev_pool = build(best_cp)
            first_loss = warm(tr, dev_pool, a.warmup)
        else:
            first_loss = ok[best]["loss_first_step"]
            warm(tr, dev_pool, max(0, a.warmup - trial_warm - trial_steps))
        cp = best_cp
    else:
        cp = cands[0]
        first_loss = warm(tr, dev_pool, a.warmup)
    targs = tr.args
    n_mb = targs.num_micro_batches
    bytes_h2d_per_mb = sum(v.numel() * v.element_size() for v in host[0].values())
    torch.cuda.reset_peak_memory_stats()
    clk_path = os.path.join(clock_log_dir(), f"bench_clocks_rank{rank}.csv")
    proc, fh = clock_sampler_start(clk_path) if rank == 0 else (None, None)
    ms_dev, launches, _ = timed(tr, dev_pool, a.steps, read_loss=False)
    clocks = clock_sampler_stop(proc, fh, clk_path, local) if rank == 0 else {}
    ms_e2e, _, last_loss = timed(tr, host, a.steps, read_loss=True)
    _lib.check_status()
    peak = torch.tensor([torch.cuda.max_memory_allocated(tr.device) / 2 ** 30], dtype=torch.float64, device=tr.device)
    if world > 1:
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
    tokens = gbs * tok_sample * a.steps
    value = tokens / (ms_dev * 1e-3)
    e2e = tokens / (ms_e2e * 1e-3)
    if rank == 0:
        inner = getattr(tr.model, "module", tr.model)
        cfg = inner.cfg
        if hunyuan:
            desc = (f"{a.model} ({cfg.num_layers} dual + {cfg.num_single_layers} single blocks, hidden {cfg.hidden_size}, "
                    f"{cfg.num_attention_heads}x{cfg.attention_head_dim} heads)")
        else:
            desc = (f"{a.model} ({cfg.num_layers} layers, dim {cfg.dim}, {cfg.num_heads}x{cfg.dim // cfg.num_heads} "
                    f"heads, ffn {cfg.ffn_dim})")
        if headline:
            metric, published = METRIC, PUBLISHED_TOKENS_PER_S_PER_GPU
            desc = "Wan2.1-1.3B t2v (30 layers, dim 1536, 12x128 heads, ffn 8960)"
        else:
            metric = f"{a.model.replace('-', '_')}_{height}p{frames}f_train_tokens_per_s"
            published = {(480, 832, 81): PUBLISHED_TOKENS_PER_S_PER_GPU,
                         (720, 1280, 81): PUBLISHED_720P_TOKENS_PER_S_PER_GPU}.get((height, width, frames))
        if a.layers:
            desc = f"{a.model} truncated to {a.layers} layers (NOT the named config)"
        fused_opt = bool(getattr(tr.optimizer, "fused", False))
        fused_cp = bool(getattr(getattr(inner, "cp", None), "fused", None))
        res = {
            "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": a.warmup, "ms_per_step": ms_dev / a.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": value / (published * world) if published else None, "dtype": "bf16", "data": "synthetic",
            "impl": "teletron_b200",
            "config": {"model": desc,
                       "global_batch": gbs, "seq_len": tok_sample,
                       "parallelism": layout_name(world, cp, tp), "micro_batches_per_step": n_mb,
                       "layout_choice": ("the fastest of `layouts` (3 + 3 step trials of every Ulysses size that "
                                         "divides the GPUs)" if len(cands) > 1 else "only candidate"),
                       "optimizer": "AdamW fp32 master" + (" (sharded)" if world > 1 else ""),
                       "grad_reduce_overlap": bool(getattr(tr.optimizer, "overlap", False)),
                       "recompute": "full" if a.recompute else "none",
                       "comm": ("peer-memory fused kernels" if (fused_opt or fused_cp) else ("nccl" if world > 1 else "none")),
                       "l2": "inputs and working set far larger than L2 (each step touches > 50 GB)",
                       "baseline_note": "vs_baseline divides by the tokens/s/GPU read off the reference's H800 chart "
                                        "(1.09k at 480P x 81, 0.57k at 720P x 81; model size not stated there)"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / a.steps,
                    "h2d_bytes_per_step": bytes_h2d_per_mb * gbs, "d2h_bytes_per_step": 4 * world,
                    "last_loss": last_loss},
            "parity": {"loss_first_step": first_loss,
                       "note": "loss of the first optimizer step: same initial weights and the same 8 samples (data, "
                               "noise and timestep are functions of the global sample index) at every N and layout"},
            "gpu_launches": launches,
            "peak_mem_gib": round(float(peak.item()), 2),   # torch allocator high-water mark, max over ranks
        }
        if layouts:
            res["layouts"] = layouts
        print(json.dumps(res), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------ reference
REF_SHAPES = {  # hidden, heads, layers, ffn (the public Wan2.1 checkpoints' shapes)
    "wan2.1-1.3b": (1536, 12, 30, 8960),
    "wan2.1-14b": (5120, 40, 40, 13824),
}


class _Stopwatch:
    """CUDA events on a GPU; the host clock when the arm is driven on CPU by the tests."""

    def __init__(self, torch, dev):
        self.torch, self.cuda = torch, dev.type == "cuda"

    def start(self):
        if self.cuda:
            self.torch.cuda.synchronize()
            self.e0 = self.torch.cuda.Event(enable_timing=True)
            self.e1 = self.torch.cuda.Event(enable_timing=True)
            self.e0.record()
        else:
            self.t0 = time.perf_counter()

    def stop_ms(self):
        if self.cuda:
            self.e1.record()
            self.torch.cuda.synchronize()
            return self.e0.elapsed_time(self.e1)
        return (time.perf_counter() - self.t0) * 1e3


def reference_result(a, *, tok_sample, gbs, desc, ms_dev, ms_e2e, e2e_steps, h2d_bytes_per_step, clocks, last_loss,
                     recompute, settings_tried):
    """The reference arm's JSON line, built from plain numbers (unit-tested without a GPU)."""
    headline = (a.model == "wan2.1-1.3b-t2v" and (a.frames, a.height, a.width, gbs) == (FRAMES, HEIGHT, WIDTH, GLOBAL_BATCH)
                and not a.layers)
    published = {(480, 832, 81): PUBLISHED_TOKENS_PER_S_PER_GPU,
                 (720, 1280, 81): PUBLISHED_720P_TOKENS_PER_S_PER_GPU}.get((a.height, a.width, a.frames))
    metric = METRIC if headline else f"{a.model.replace('-', '_')}_{a.height}p{a.frames}f_train_tokens_per_s"
    value = gbs * tok_sample * a.steps / (ms_dev * 1e-3)
    e2e = gbs * tok_sample * e2e_steps / (ms_e2e * 1e-3)
    return {
        "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": a.steps, "warmup": a.warmup,
        "ms_per_step": ms_dev / a.steps, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": value / published if published else None, "dtype": "bf16", "data": "synthetic",
        "impl": "reference",
        "config": {"model": desc, "global_batch": gbs, "seq_len": tok_sample, "parallelism": "dp1",
                   "micro_batches_per_step": gbs, "optimizer": "torch fused AdamW on bf16 parameters",
                   "recompute": recompute, "recompute_settings_tried": settings_tried,
                   "l2": "inputs and working set far larger than L2",
                   "note": "unmodified teletron/models/wan/wan_model.py + flow_match.py from baseline/_ref, flash_attn 2 "
                           "attention; the reference Trainer itself cannot be imported offline (megatron-core, apex, "
                           "yunchang missing)"},
        "clocks": clocks,
        "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / e2e_steps, "steps": e2e_steps,
                "h2d_bytes_per_step": h2d_bytes_per_step, "d2h_bytes_per_step": 4, "last_loss": last_loss},
    }


def run_reference(a, device=None, shape=None, ref_root=None, time_budget_s=1500.0):
    """The reference's own DiT code from baseline/_ref, driven directly: its Trainer needs
    megatron-core / apex / yunchang, none of which can be installed offline.

    One step = `--global-batch` micro-batches of one sample through the reference's `WanModel.forward`
    (`teletron/models/wan/wan_model.py:339-396`) with the flow-matching loss of its example
    (`examples/wan/pretrain_wan.py:26-62`), gradient clipping and one AdamW step.  Both of its activation settings are
    tried for two steps (per-block checkpointing as shipped, and none); the faster one that fits is measured and
    named in `config.recompute`.  `device` / `shape` / `ref_root` exist for the CPU test of this function."""
    rank, world, local = dist_env()
    t_wall0 = time.time()

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
        return 0

    ref_root = Path(ref_root) if ref_root else ROOT / "baseline" / "_ref"
    ref_file = ref_root / "teletron" / "models" / "wan" / "wan_model.py"
    if not ref_file.exists():
        return unavailable("reference not installed under baseline/_ref (pip --no-deps install missing)")
    if world > 1 or a.gpus > 1:
        return unavailable("multi-GPU reference path needs megatron-core 0.6.0 + yunchang (parallel_state, DDP, "
                           "Ulysses all-to-all); neither is in the offline wheelhouse, so only N=1 runs")
    key = a.model.rsplit("-", 1)[0]
    if key not in REF_SHAPES and shape is None:
        return unavailable(f"the reference has no model named {a.model}")
    import importlib.util
    from types import SimpleNamespace

    import torch

    if device is None and not torch.cuda.is_available():
        return unavailable("no CUDA device on this machine")
    spec = importlib.util.spec_from_file_location("ref_wan_model", ref_file)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    fm_spec = importlib.util.spec_from_file_location("ref_flow_match", ref_file.parent.parent / "flow_match.py")
    fm = importlib.util.module_from_spec(fm_spec)
    fm_spec.loader.exec_module(fm)
    dev = torch.device(device) if device is not None else torch.device("cuda", local)
    on_gpu = dev.type == "cuda"
    if on_gpu:
        torch.cuda.set_device(dev)
    else:  # CPU test: the flash-attention wheels cannot take CPU tensors
        ref.FLASH_ATTN_3_AVAILABLE = ref.FLASH_ATTN_2_AVAILABLE = ref.SAGE_ATTN_AVAILABLE = False
    hidden, heads, layers, ffn = shape["dims"] if shape else REF_SHAPES[key]
    text_dim, text_len = (shape["text_dim"], shape["text_len"]) if shape else (4096, 512)
    i2v = "i2v" in a.model
    P = ref.WanParams  # model shape is class-level configuration in the reference
    P.in_channels, P.ffn_dim, P.has_image_input, P.text_dim = (36 if i2v else 16), ffn, i2v, text_dim
    if shape:
        P.freq_dim = shape.get("freq_dim", P.freq_dim)
    n_layers = a.layers or layers
    gbs = a.global_batch
    tok_sample = tokens_per_sample(a.frames, a.height, a.width)
    dtype = torch.bfloat16 if on_gpu else torch.float32
    torch.manual_seed(1234)
    model = ref.WanModel(SimpleNamespace(hidden_size=hidden, num_attention_heads=heads, num_layers=n_layers))
    model = model.to(dev).to(dtype).train()
    opt = torch.optim.AdamW(model.parameters(), lr=1e-5, weight_decay=1e-2, fused=on_gpu)
    sched = fm.FlowMatchScheduler(shift=5, sigma_min=0.0, extra_one_step=True)
    sched.set_timesteps(1000, training=True)
    f, h, w = (a.frames - 1) // 4 + 1, a.height // 8, a.width // 8

    def sample(g):
        b = dict(latents=torch.randn(1, 16, f, h, w, generator=g).to(dtype),
                 context=torch.randn(1, text_len, text_dim, generator=g).to(dtype))
        if i2v:
            b["clip_feature"] = torch.randn(1, 257, 1280, generator=g).to(dtype)
            b["y"] = torch.randn(1, 20, f, h, w, generator=g).to(dtype)
        return {k: (v.pin_memory() if on_gpu else v) for k, v in b.items()}

    g = torch.Generator().manual_seed(1234)
    pool_host = [sample(g) for _ in range(min(gbs, 8))]
    pool_dev = [{k: v.to(dev) for k, v in b.items()} for b in pool_host]
    h2d_per_mb = sum(v.numel() * v.element_size() for v in pool_host[0].values())

    def step(pool, use_ckpt, copy_in):
        opt.zero_grad(set_to_none=True)
        for mb in range(gbs):
            b = pool[mb % len(pool)]
            if copy_in:  # this micro-batch's inputs come from pinned host memory
                b = {k: v.to(dev, non_blocking=True) for k, v in b.items()}
            latents = b["latents"]
            noise = torch.randn_like(latents)
            tid = torch.randint(0, sched.num_train_timesteps, (1,))
            timestep = sched.timesteps[tid].to(dtype=dtype, device=dev)
            target = sched.training_target(latents, noise, timestep)
            noisy = sched.add_noise(latents, noise, timestep)
            out = model(x=noisy, timestep=timestep, context=b["context"], clip_feature=b.get("clip_feature"),
                        y=b.get("y"), use_gradient_checkpointing=use_ckpt)
            loss = torch.nn.functional.mse_loss(out.float(), target.float()) * sched.training_weight(timestep)
            (loss / gbs).backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        return loss

    oom = torch.cuda.OutOfMemoryError if on_gpu else MemoryError
    watch = _Stopwatch(torch, dev)
    # two steps of each activation setting; the second one is timed
    candidates = [False] if a.ref_no_recompute else ([True] if a.ref_recompute_only else [True, False])
    tried, probe_ms = {}, {}
    for use_ckpt in candidates:
        name = "per-block checkpointing (the reference's shipped setting)" if use_ckpt else "none"
        try:
            step(pool_dev, use_ckpt, False)
            watch.start()
            step(pool_dev, use_ckpt, False)
            probe_ms[use_ckpt] = watch.stop_ms()
            tried[name] = f"{probe_ms[use_ckpt]:.0f} ms/step"
        except oom:
            tried[name] = "out of memory"
            opt.zero_grad(set_to_none=True)
            if on_gpu:
                torch.cuda.empty_cache()
    if not probe_ms:
        return unavailable("reference model ran out of memory in warm-up with every activation setting")
    use_ckpt = min(probe_ms, key=probe_ms.get)
    recompute = "per-block checkpointing (the reference's shipped setting)" if use_ckpt else "none"
    for _ in range(max(0, a.warmup - 2)):
        step(pool_dev, use_ckpt, False)
    clk_path = os.path.join(clock_log_dir(), "bench_clocks_reference.csv")
    proc, fh = clock_sampler_start(clk_path) if on_gpu else (None, None)
    watch.start()
    for _ in range(a.steps):
        step(pool_dev, use_ckpt, False)
    ms_dev = watch.stop_ms()
    clocks = clock_sampler_stop(proc, fh, clk_path, local)
    # end to end: inputs from pinned host memory every micro-batch, the loss read back every step; fewer steps
    # only if the whole arm would otherwise outrun its time budget (said in e2e.steps)
    per_step_s = ms_dev * 1e-3 / a.steps
    left = time_budget_s - (time.time() - t_wall0)
    e2e_steps = max(1, min(a.steps, int(left / max(per_step_s, 1e-9))))
    last_loss = None
    watch.start()
    for _ in range(e2e_steps):
        last_loss = float(step(pool_host, use_ckpt, True).detach())
    ms_e2e = watch.stop_ms()
    desc = f"{a.model} ({n_layers} layers, dim {hidden}, {heads}x{hidden // heads} heads, ffn {ffn})"
    if a.layers:
        desc += " truncated (NOT the named config)"
    print(json.dumps(reference_result(
        a, tok_sample=tok_sample, gbs=gbs, desc=desc, ms_dev=ms_dev, ms_e2e=ms_e2e, e2e_steps=e2e_steps,
        h2d_bytes_per_step=h2d_per_mb * gbs, clocks=clocks, last_loss=last_loss, recompute=recompute,
        settings_tried=tried)), flush=True)
    return 0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", type=str, default="wan2.1-1.3b-t2v")
    ap.add_argument("--cp", type=int, default=0, help="Ulysses context-parallel size, the rest is DP (0: measure every "
                                                       "size that divides the GPUs, report all, headline = the fastest)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel size (HunyuanVideo)")
    ap.add_argument("--no-overlap", action="store_true", help="reduce gradients after backward instead of during it")
    ap.add_argument("--recompute", action="store_true", help="full activation recompute (not needed at 1.3B)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: truncate the model (invalid as a result)")
    ap.add_argument("--frames", type=int, default=FRAMES)
    ap.add_argument("--height", type=int, default=HEIGHT)
    ap.add_argument("--width", type=int, default=WIDTH)
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH)
    ap.add_argument("--init-on-device", action="store_true", help="create parameters on the GPU (default for 14B)")
    ap.add_argument("--ref-no-recompute", action="store_true", help="reference arm: only the no-checkpointing setting")
    ap.add_argument("--ref-recompute-only", action="store_true", help="reference arm: only per-block checkpointing")
    ap.add_argument("--fused-comm", type=str, default="auto", choices=["auto", "on", "off"],
                    help="peer-memory fused collectives (off = NCCL baseline path)")
    a = ap.parse_args(argv)
    if a.impl == "reference":
        sys.exit(run_reference(a) or 0)
    run_ours(a)


if __name__ == "__main__":
    main()
