"""Name -> class registries for models and encoders.

Small counterpart of teletron/models/registry.py:37-240, teletron/models/build.py:8-16 and
teletron/models/encoder_registry.py:9-56: ``build_model(name, config)`` returns a model
instance, ``get_encoder(name, device)`` an encoder, ``MODEL_TO_ENCODER`` maps a model name to
the encoder that feeds it.
"""
from __future__ import annotations

from typing import Callable, Dict


class Registry:
    def __init__(self, kind: str):
        self.kind = kind
        self._items: Dict[str, Callable] = {}

    def register(self, name: str = None):
        def deco(obj):
            key = name or obj.__name__
            if key in self._items and self._items[key] is not obj:
                raise KeyError(f"{self.kind} {key!r} is already registered")
            self._items[key] = obj
            return obj

        return deco

    def get(self, name: str):
        if name not in self._items:
            raise KeyError(f"unknown {self.kind} {name!r}; known: {sorted(self._items)}")
        return self._items[name]

    def __contains__(self, name):
        return name in self._items

    def names(self):
        return sorted(self._items)


MODELS = Registry("model")
ENCODERS = Registry("encoder")
# HunyuanVideo: the reference ships no encoder bundle for it; the weight-free stand-in serves the schema until a
# user-supplied BaseEncoder subclass is named with --encoder-name
MODEL_TO_ENCODER = {"ParallelWanModel": "wan_encoder", "WanModel": "wan_encoder",
                    "ParallelHunyuanVideoModel": "synthetic_hunyuan_encoder",
                    "HunyuanVideoModel": "synthetic_hunyuan_encoder"}


def build_model(name: str, config, **kw):
    return MODELS.get(name)(config, **kw)


def get_encoder(name: str, device=None, **kw):
    return ENCODERS.get(name)(device=device, **kw)


def encoder_for_model(model_name: str) -> str:
    return MODEL_TO_ENCODER[model_name]
