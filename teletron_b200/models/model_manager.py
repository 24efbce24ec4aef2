"""Loading checkpoints from disk into models: file reading (.safetensors / .pth / .ckpt / .bin,
sharded lists), model-type detection and meta-device instantiation with ``assign=True`` loading.

Counterpart of the reference ModelManager and its helpers (teletron/models/wan/encoder/
model_manager.py:13-415, wan_encoder_utils.py:232-368).  Detection is by characteristic keys /
shapes instead of key-hash tables; the Wan DiT accepts native, diffusers and prefixed layouts.
``load_lora`` folds low-rank adapter files (PEFT ``lora_A`` / ``lora_B`` or kohya ``lora_down`` /
``lora_up`` naming, optional per-module ``alpha``) into the weights of a loaded model, so inference
and further training run on the fused kernels unchanged (the reference's ``load_lora``, model_manager.py:
333-353, depends on loaders that are not in its tree).
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


_CONSTANT_BUFFERS = ("mean", "std", "inv_std")   # normalisation constants set by the module itself, never in a file


def align_checkpoint_keys(module: torch.nn.Module, sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Checkpoint files of the encoders come without the wrapper prefix the module classes use (the CLIP and VAE
    files store ``visual.*`` / ``encoder.*`` while the modules hold them under ``model.``; the CLIP file also carries
    the unused text tower and ``log_scale``).  Returns the entries of ``sd`` renamed to the spelling (as is,
    ``model.`` added, ``model.`` removed) that matches most of ``module``'s keys, dropping entries the module does not
    have (the reference does this per model in its ``from_civitai`` converters, wan_video_image_encoder.py:889-904)."""
    want = set(module.state_dict().keys())
    spellings = (sd, {"model." + k: v for k, v in sd.items()},
                 {k[len("model."):]: v for k, v in sd.items() if k.startswith("model.")})
    best = max(spellings, key=lambda d: len(want.intersection(d)))
    return {k: v for k, v in best.items() if k in want}


@contextmanager
def init_weights_on_device(device=torch.device("meta")):
    """Construct modules without allocating / initialising real storage."""
    with torch.device(device):
        yield


_LORA_PAIRS = ((".lora_A.weight", ".lora_B.weight"), (".lora_A.default.weight", ".lora_B.default.weight"),
               (".lora_down.weight", ".lora_up.weight"))
_LORA_PREFIXES = ("base_model.model.", "diffusion_model.", "transformer.", "model.", "lora_unet_")


def is_lora_state_dict(sd: Dict[str, torch.Tensor]) -> bool:
    return any(k.endswith(down) for k in sd for down, _ in _LORA_PAIRS)


def merge_lora(model: torch.nn.Module, lora_sd: Dict[str, torch.Tensor], alpha: float = 1.0) -> List[str]:
    """``W += alpha * scale * up @ down`` for every adapter pair whose module exists in ``model``; ``scale`` is
    ``<module>.alpha / rank`` when the file carries it, else 1.  Returns the names of the updated parameters
    and raises when the file matches nothing (a wrong base model)."""
    # checkpoint-layout names: a fused projection (q, k, v stored as one matrix) appears under its separate
    # names as views of the fused storage, so the in-place update below reaches the parameter
    params = {k: v for k, v in model.state_dict().items() if torch.is_tensor(v)}
    updated = []
    for key, down in lora_sd.items():
        for d_suffix, u_suffix in _LORA_PAIRS:
            if not key.endswith(d_suffix):
                continue
            stem = key[: -len(d_suffix)]
            up = lora_sd.get(stem + u_suffix)
            if up is None:
                raise KeyError(f"{key} has no matching {stem + u_suffix}")
            name = stem
            for pre in _LORA_PREFIXES:
                if name.startswith(pre) and (name[len(pre):] + ".weight") in params:
                    name = name[len(pre):]
                    break
            target = params.get(name + ".weight")
            if target is None:
                continue
            rank = down.shape[0]
            scale = float(lora_sd[stem + ".alpha"]) / rank if (stem + ".alpha") in lora_sd else 1.0
            delta = (up.float().flatten(1) @ down.float().flatten(1)) * (alpha * scale)
            if delta.numel() != target.numel():
                raise ValueError(f"adapter for {name} has shape {tuple(delta.shape)}, weight is {tuple(target.shape)}")
            with torch.no_grad():
                target.add_(delta.view_as(target).to(device=target.device, dtype=target.dtype))
            updated.append(name + ".weight")
    if not updated:
        raise ValueError("no adapter in the file matches a module of this model")
    return updated


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
        if isinstance(path, str) and os.path.isdir(path):     # a folder of shards counts as one checkpoint
            shards = sorted(os.path.join(path, f) for f in os.listdir(path)
                            if f.endswith((".safetensors", ".pth", ".pt", ".bin", ".ckpt")))
            if not shards:
                raise FileNotFoundError(f"no weight files in {path}")
            path = shards
        sd = load_state_dict(path, "cpu", dt)
        kind = detect_model_type(sd)
        if kind is None:
            raise ValueError(f"cannot tell what model {path} holds ({len(sd)} tensors)")
        model = self._instantiate(kind, sd)
        use = self._wan_sd if kind == "wan_video_dit" else align_checkpoint_keys(model, sd)
        missing, unexpected = model.load_state_dict(use, assign=True, strict=False)
        missing = [k for k in missing if k.split(".")[-1] not in _CONSTANT_BUFFERS]
        if missing:
            raise RuntimeError(f"{path}: {len(missing)} parameters missing, e.g. {missing[:3]}")
        if hasattr(model, "reset_constants"):        # constants built on the meta device hold no values
            model.reset_constants("cpu")
        stale = [n for n, b in model.named_buffers() if b.is_meta]
        if stale:
            raise RuntimeError(f"{path}: buffers {stale[:3]} of {type(model).__name__} were built on the meta device "
                               "and are set by neither the file nor reset_constants()")
        self.models[kind] = model.to(device=device).eval()
        self.paths[kind] = path
        return self.models[kind]

    def load_models(self, paths, device=None, torch_dtype=None):
        for p in paths:
            self.load_model(p, device, torch_dtype)

    def load_lora(self, path=None, state_dict=None, lora_alpha: float = 1.0, kind: Optional[str] = None):
        """Fold an adapter file into a loaded model: ``kind`` if given, else the first loaded model it matches."""
        sd = state_dict if state_dict is not None else load_state_dict(path, "cpu")
        if not is_lora_state_dict(sd):
            raise ValueError(f"{path or 'state dict'} holds no low-rank adapter weights")
        for k in ([kind] if kind else list(self.models)):
            try:
                return k, merge_lora(self.models[k], sd, lora_alpha)
            except ValueError:
                if kind:
                    raise
        raise ValueError("the adapter matches none of the loaded models")

    def to(self, device):
        for k, m in self.models.items():
            self.models[k] = m.to(device)
        self.device = device
        return self

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
