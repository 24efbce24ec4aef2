"""Weight import for the Wan DiT: diffusers -> native key names and model-shape detection.

The reference renames keys through a per-block lookup table and recognises variants by an md5 of
the sorted key list (teletron/models/wan/converter.py:7-228, wan_model_config.py:11-44).  Here the
renames are pattern rules and the configuration is read from the tensor shapes themselves
(dim, layers, ffn, heads = dim / 128, input channels, image branch), which also covers variants
that no hash table lists.  ``hash_state_dict_keys`` is kept for callers that key on it.
"""
from __future__ import annotations

import hashlib
import re
from typing import Dict, Tuple

import torch

from .wan import WanConfig

_RULES = [
    (r"^blocks\.(\d+)\.attn1\.to_(q|k|v)\.(weight|bias)$", r"blocks.\1.self_attn.\2.\3"),
    (r"^blocks\.(\d+)\.attn1\.to_out\.0\.(weight|bias)$", r"blocks.\1.self_attn.o.\2"),
    (r"^blocks\.(\d+)\.attn1\.norm_(q|k)\.weight$", r"blocks.\1.self_attn.norm_\2.weight"),
    (r"^blocks\.(\d+)\.attn2\.to_(q|k|v)\.(weight|bias)$", r"blocks.\1.cross_attn.\2.\3"),
    (r"^blocks\.(\d+)\.attn2\.to_out\.0\.(weight|bias)$", r"blocks.\1.cross_attn.o.\2"),
    (r"^blocks\.(\d+)\.attn2\.norm_(q|k)\.weight$", r"blocks.\1.cross_attn.norm_\2.weight"),
    (r"^blocks\.(\d+)\.attn2\.add_(k|v)_proj\.(weight|bias)$", r"blocks.\1.cross_attn.\2_img.\3"),
    (r"^blocks\.(\d+)\.attn2\.norm_added_k\.weight$", r"blocks.\1.cross_attn.norm_k_img.weight"),
    (r"^blocks\.(\d+)\.ffn\.net\.0\.proj\.(weight|bias)$", r"blocks.\1.ffn.0.\2"),
    (r"^blocks\.(\d+)\.ffn\.net\.2\.(weight|bias)$", r"blocks.\1.ffn.2.\2"),
    (r"^blocks\.(\d+)\.norm2\.(weight|bias)$", r"blocks.\1.norm3.\2"),
    (r"^blocks\.(\d+)\.scale_shift_table$", r"blocks.\1.modulation"),
    (r"^condition_embedder\.text_embedder\.linear_1\.(weight|bias)$", r"text_embedding.0.\1"),
    (r"^condition_embedder\.text_embedder\.linear_2\.(weight|bias)$", r"text_embedding.2.\1"),
    (r"^condition_embedder\.time_embedder\.linear_1\.(weight|bias)$", r"time_embedding.0.\1"),
    (r"^condition_embedder\.time_embedder\.linear_2\.(weight|bias)$", r"time_embedding.2.\1"),
    (r"^condition_embedder\.time_proj\.(weight|bias)$", r"time_projection.1.\1"),
    (r"^condition_embedder\.image_embedder\.norm1\.(weight|bias)$", r"img_emb.proj.0.\1"),
    (r"^condition_embedder\.image_embedder\.ff\.net\.0\.proj\.(weight|bias)$", r"img_emb.proj.1.\1"),
    (r"^condition_embedder\.image_embedder\.ff\.net\.2\.(weight|bias)$", r"img_emb.proj.3.\1"),
    (r"^condition_embedder\.image_embedder\.norm2\.(weight|bias)$", r"img_emb.proj.4.\1"),
    (r"^patch_embedding\.(weight|bias)$", r"patch_embedding.\1"),
    (r"^scale_shift_table$", r"head.modulation"),
    (r"^proj_out\.(weight|bias)$", r"head.head.\1"),
]
_COMPILED = [(re.compile(p), r) for p, r in _RULES]


def hash_state_dict_keys(state_dict: Dict[str, torch.Tensor], with_shape: bool = True) -> str:
    """md5 over the sorted ``name[:shape]`` list (teletron/models/wan/encoder/wan_encoder_utils.py:232-368)."""
    parts = []
    for k in sorted(state_dict):
        v = state_dict[k]
        parts.append(f"{k}:{'_'.join(map(str, v.shape))}" if (with_shape and torch.is_tensor(v)) else k)
    return hashlib.md5(",".join(parts).encode()).hexdigest()


def is_diffusers_layout(state_dict) -> bool:
    return any(k.startswith("condition_embedder.") or ".attn1." in k for k in state_dict)


def from_diffusers(state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in state_dict.items():
        k = k[len("model.diffusion_model."):] if k.startswith("model.diffusion_model.") else k
        for pat, rep in _COMPILED:
            if pat.match(k):
                out[pat.sub(rep, k)] = v
                break
    return out


def from_civitai(state_dict):
    """Single-file community checkpoints: native names, possibly under a ``model.diffusion_model.`` prefix."""
    pre = "model.diffusion_model."
    return {(k[len(pre):] if k.startswith(pre) else k): v for k, v in state_dict.items()}


def detect_wan_config(state_dict: Dict[str, torch.Tensor], head_dim: int = 128) -> WanConfig:
    """Read the model shape off a native-layout state dict."""
    pe = state_dict["patch_embedding.weight"]
    dim, in_dim = pe.shape[0], pe.shape[1]
    layers = 1 + max(int(k.split(".")[1]) for k in state_dict if k.startswith("blocks."))
    ffn = state_dict["blocks.0.ffn.0.weight"].shape[0]
    text_dim = state_dict["text_embedding.0.weight"].shape[1]
    freq_dim = state_dict["time_embedding.0.weight"].shape[1]
    out_dim = state_dict["head.head.weight"].shape[0] // 4
    has_img = any(k.startswith("img_emb.") for k in state_dict)
    return WanConfig(dim=dim, num_heads=dim // head_dim, num_layers=layers, ffn_dim=ffn, in_dim=in_dim,
                     out_dim=out_dim, text_dim=text_dim, freq_dim=freq_dim, has_image_input=has_img,
                     has_image_pos_emb="img_emb.emb_pos" in state_dict)


def convert_wan_state_dict(state_dict) -> Tuple[Dict[str, torch.Tensor], WanConfig]:
    sd = from_diffusers(state_dict) if is_diffusers_layout(state_dict) else from_civitai(state_dict)
    return sd, detect_wan_config(sd)


# ------------------------------------------------------------------------------------- command line
def write_release_checkpoint(state_dict: Dict[str, torch.Tensor], out_dir: str, dtype=torch.bfloat16) -> str:
    """Write ``state_dict`` (native names) as a Megatron-layout checkpoint the trainer loads with ``--load`` or
    ``--pretrained-checkpoint``: ``<out>/release/mp_rank_00/model_optim_rng.pt`` plus a tracker file that says
    ``release`` (weights only: iteration 0, no optimizer state)."""
    import os

    path = os.path.join(out_dir, "release", "mp_rank_00", "model_optim_rng.pt")
    os.makedirs(os.path.dirname(path), exist_ok=True)
    sd = {k: (v.to(dtype) if torch.is_tensor(v) and v.is_floating_point() else v) for k, v in state_dict.items()}
    tmp = path + ".tmp"
    torch.save(dict(model=sd, checkpoint_version=3.0, iteration=0), tmp)
    os.replace(tmp, path)
    with open(os.path.join(out_dir, "latest_checkpointed_iteration.txt"), "w") as f:
        f.write("release")
    return path


def main(argv=None) -> int:
    """``python -m teletron_b200.models.convert --input <file | shard ... | folder> --output <dir>``: read a Wan DiT
    checkpoint in diffusers, community single-file or native naming, report the detected shape and write it in the
    trainer's checkpoint layout."""
    import argparse

    from .model_manager import load_state_dict

    ap = argparse.ArgumentParser(description=main.__doc__)
    ap.add_argument("--input", nargs="+", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32"])
    a = ap.parse_args(argv)
    import os

    paths = a.input
    if len(paths) == 1 and os.path.isdir(paths[0]):
        paths = sorted(os.path.join(paths[0], f) for f in os.listdir(paths[0])
                       if f.endswith((".safetensors", ".pth", ".pt", ".bin", ".ckpt")))
    sd, cfg = convert_wan_state_dict(load_state_dict(paths if len(paths) > 1 else paths[0]))
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}[a.dtype]
    out = write_release_checkpoint(sd, a.output, dtype)
    n = sum(v.numel() for v in sd.values() if torch.is_tensor(v))
    print(f"Wan DiT: dim {cfg.dim}, {cfg.num_layers} layers, {cfg.num_heads} heads, ffn {cfg.ffn_dim}, in {cfg.in_dim}, "
          f"image branch {cfg.has_image_input}; {n / 1e9:.3f} B parameters ({hash_state_dict_keys(sd)}) -> {out}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
