"""``ParallelWanModel``: the registered training model = WanModel + Ulysses context + recompute
policy taken from the trainer's arguments (teletron/models/wan/parallel_wan_model.py:40-124).

``config`` may be a ``WanConfig`` or any namespace with Megatron-style fields
(``hidden_size``, ``num_attention_heads``, ``num_layers``, ``ffn_hidden_size``,
``recompute_*``, ``activation_offload``, ``task_type``), which is how the reference passes model
shape (teletron/train/utils.py:907-948).
"""
from __future__ import annotations

from ..parallel import state as mpu
from ..parallel.ulysses import UlyssesContext
from .registry import MODELS
from .wan import WAN_PRESETS, WanConfig, WanModel


def config_from_args(a) -> WanConfig:
    if isinstance(a, WanConfig):
        return a
    preset = getattr(a, "model_preset", None)
    kw = dict(WAN_PRESETS[preset]) if preset else {}
    task = getattr(a, "task_type", None) or ("i2v" if kw.get("has_image_input") else "t2v")
    if getattr(a, "hidden_size", None):
        kw["dim"] = a.hidden_size
    if getattr(a, "num_attention_heads", None):
        kw["num_heads"] = a.num_attention_heads
    if getattr(a, "num_layers", None):
        kw["num_layers"] = a.num_layers
    if getattr(a, "ffn_hidden_size", None):
        kw["ffn_dim"] = a.ffn_hidden_size
    elif "ffn_dim" not in kw:
        kw["ffn_dim"] = {1536: 8960, 5120: 13824}.get(kw.get("dim", 1536), 4 * kw.get("dim", 1536))
    if "in_dim" not in kw or getattr(a, "task_type", None):
        kw["in_dim"] = 36 if task == "i2v" else 16
        kw["has_image_input"] = task == "i2v"
    for f in ("text_dim", "freq_dim"):
        if getattr(a, f, None):
            kw[f] = getattr(a, f)
    kw["recompute_granularity"] = getattr(a, "recompute_granularity", None)
    kw["recompute_method"] = getattr(a, "recompute_method", None) or "block"
    kw["recompute_num_layers"] = getattr(a, "recompute_num_layers", None) or 0
    kw["activation_offload"] = bool(getattr(a, "activation_offload", False))
    return WanConfig(**kw)


@MODELS.register("ParallelWanModel")
class ParallelWanModel(WanModel):
    def __init__(self, config, cp: UlyssesContext = None, **_):
        cfg = config_from_args(config)
        if cp is None and mpu.model_parallel_is_initialized() and mpu.get_context_parallel_world_size() > 1:
            cp = UlyssesContext(mpu.get_context_parallel_group(), mpu.get_context_parallel_world_size(),
                                mpu.get_context_parallel_rank())
        super().__init__(cfg, cp)

    # the reference exposes these for its checkpoint code (parallel_wan_model.py:119-124)
    def state_dict_for_save_checkpoint(self, prefix="", keep_vars=False):
        return self.state_dict(prefix=prefix, keep_vars=keep_vars)

    def sharded_state_dict(self, prefix=""):
        return self.state_dict(prefix=prefix)

    def set_input_tensor(self, input_tensor):  # pipeline parallelism hook; PP = 1 only
        return None


MODELS.register("WanModel")(WanModel)
