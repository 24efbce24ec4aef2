"""Loading checkpoints from disk into models: file reading (.safetensors / .pth / .ckpt / .bin,
sharded lists), model-type detection and meta-device instantiation with ``assign=True`` loading.

Counterpart of the reference ModelManager and its helpers (teletron/models/wan/encoder/
model_manager.py:13-415, wan_encoder_utils.py:232-368).  Detection is by characteristic keys /
shapes instead of key-hash tables; the Wan DiT accepts native, diffusers and prefixed layouts.
"""
from __future__ import annotations

import os
from contextlib import contextmanager
from typing import Dict, List, Optional, Union

import torch

from .convert import convert_wan_state_dict


def load_state_dict(path: Union[str, List[str]], device="cpu", torch_dtype=None) -> Dict[str, torch.Tensor]:
    if isinstance(path, (list, tuple)):
        out = {}
        for p in path:
            out.update(load_state_dict(p, device, torch_dtype))
        return out
    if path.endswith(".safetensors"):
        from safetensors import safe_open

        sd = {}
        with safe_open(path, framework="pt", device=str(device)) as f:
            for k in f.keys():
                sd[k] = f.get_tensor(k)
    else:
        sd = torch.load(path, map_location=device, weights_only=True)
        for wrap in ("state_dict", "model_state", "module", "model"):
            if isinstance(sd, dict) and wrap in sd and isinstance(sd[wrap], dict):
                sd = sd[wrap]
    if torch_dtype is not None:
        sd = {k: (v.to(torch_dtype) if torch.is_tensor(v) and v.is_floating_point() else v) for k, v in sd.items()}
    return sd


@contextmanager
def init_weights_on_device(device=torch.device("meta")):
    """Construct modules without allocating / initialising real storage."""
    with torch.device(device):
        yield


def detect_model_type(sd: Dict[str, torch.Tensor]) -> Optional[str]:
    keys = sd.keys()
    if any(k.endswith("patch_embedding.weight") for k in keys) and any("self_attn" in k or ".attn1." in k for k in keys):
        return "wan_video_dit"
    if any(k.startswith("token_embedding.") for k in keys) and any(".pos_embedding.embedding" in k for k in keys):
        return "wan_video_text_encoder"
    if any("visual.transformer" in k for k in keys):
        return "wan_video_image_encoder"
    if any(k.startswith(("encoder.downsamples", "model.encoder.downsamples")) for k in keys):
        return "wan_video_vae"
    if any(k.startswith("single_transformer_blocks.") for k in keys):
        return "hunyuan_video_dit"
    return None


class ModelManager:
    def __init__(self, torch_dtype=torch.bfloat16, device="cpu"):
        self.torch_dtype, self.device = torch_dtype, device
        self.models: Dict[str, torch.nn.Module] = {}
        self.paths: Dict[str, object] = {}

    def load_model(self, path, device=None, torch_dtype=None):
        device, dt = device or self.device, torch_dtype or self.torch_dtype
        sd = load_state_dict(path, "cpu", dt)
        kind = detect_model_type(sd)
        if kind is None:
            raise ValueError(f"cannot tell what model {path} holds ({len(sd)} tensors)")
        model = self._instantiate(kind, sd)
        missing, unexpected = model.load_state_dict(sd if kind != "wan_video_dit" else self._wan_sd, assign=True,
                                                    strict=False)
        if missing:
            raise RuntimeError(f"{path}: {len(missing)} parameters missing, e.g. {missing[:3]}")
        self.models[kind] = model.to(device=device).eval()
        self.paths[kind] = path
        return self.models[kind]

    def load_models(self, paths, device=None, torch_dtype=None):
        for p in paths:
            self.load_model(p, device, torch_dtype)

    def _instantiate(self, kind, sd):
        with init_weights_on_device():
            if kind == "wan_video_dit":
                from .wan import WanModel

                self._wan_sd, cfg = convert_wan_state_dict(sd)
                return WanModel(cfg)
            if kind == "wan_video_text_encoder":
                from .encoders.umt5 import UMT5Encoder

                return UMT5Encoder()
            if kind == "wan_video_image_encoder":
                from .encoders.clip_vit import WanImageEncoder

                return WanImageEncoder()
            if kind == "wan_video_vae":
                from .encoders.wan_vae import WanVideoVAE

                return WanVideoVAE()
            if kind == "hunyuan_video_dit":
                from .hunyuan import HunyuanVideoModel, hunyuan_config

                return HunyuanVideoModel(hunyuan_config("hunyuanvideo-13b-t2v"))
        raise ValueError(kind)

    def fetch_model(self, kind: str, require: bool = False):
        m = self.models.get(kind)
        if m is None and require:
            raise KeyError(f"no {kind} loaded; have {sorted(self.models)}")
        return m
