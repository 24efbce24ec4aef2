"""Name -> class registries for models and encoders.

Small counterpart of teletron/models/registry.py:37-240, teletron/models/build.py:8-16 and
teletron/models/encoder_registry.py:9-56: ``build_model(name, config)`` returns a model
instance, ``get_encoder(name, device)`` an encoder, ``MODEL_TO_ENCODER`` maps a model name to
the encoder that feeds it.
"""
from __future__ import annotations

from typing import Callable, Dict


class Registry:
    """Name -> class table.  ``@REG.register("name")``, ``@REG.register`` (class name) and
    ``REG.register_module(cls, name)`` add entries; ``REG.build("name", config, **kw)`` or
    ``REG.build({"type": "name", ...})`` instantiate one (the two spellings of the reference's model and dataset
    registries, teletron/models/registry.py:70-190, teletron/datasets/registry.py:24-63)."""

    def __init__(self, kind: str):
        self.kind = kind
        self._items: Dict[str, Callable] = {}

    def register_module(self, obj, name: str = None):
        key = name or obj.__name__
        if key in self._items and self._items[key] is not obj:
            raise KeyError(f"{self.kind} {key!r} is already registered")
        self._items[key] = obj
        return obj

    def register(self, name=None):
        if isinstance(name, str) or name is None:
            return lambda obj: self.register_module(obj, name)
        return self.register_module(name)                     # used as a bare decorator

    def unregister(self, name: str) -> None:
        if name not in self._items:
            raise KeyError(f"unknown {self.kind} {name!r}")
        del self._items[name]

    def get(self, name: str):
        if name not in self._items:
            raise KeyError(f"unknown {self.kind} {name!r}; known: {sorted(self._items)}")
        return self._items[name]

    get_module = get

    def build(self, spec, *args, **kwargs):
        """``spec``: a registered name, or a mapping with a ``type`` key whose other items become keyword arguments
        (explicit keyword arguments win)."""
        if isinstance(spec, dict):
            params = dict(spec)
            if "type" not in params:
                raise KeyError(f"a {self.kind} spec needs a 'type' entry, got keys {sorted(params)}")
            name = params.pop("type")
            params.update(kwargs)
            return self.get(name)(*args, **params)
        return self.get(spec)(*args, **kwargs)

    def list_modules(self) -> Dict[str, Callable]:
        return dict(self._items)

    def __contains__(self, name):
        return name in self._items

    def __len__(self):
        return len(self._items)

    def __repr__(self):
        return f"Registry({self.kind}: {', '.join(sorted(self._items))})"

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
