"""Attribute-style configuration dictionary with json / yaml / pickle IO.

Counterpart of the reference's generic ``Config`` (teletron/train/config.py:20-172): nested mappings become
``Config`` objects, ``update`` merges nested mappings key by key (a ``"__force__": True`` entry replaces the
sub-tree instead), tuples survive a JSON round trip (stored as ``["__tuple__", ...]``), ``load`` / ``save`` pick
the format from the suffix, ``load_config`` accepts a path, a folder holding ``config.json``, a mapping or a
``Config``.  Python-module configs (``*.py`` / ``*.config`` paths resolved by import) are not supported: a config
file is data here, not code.
"""
from __future__ import annotations

import copy
import json
import os
import pickle
import pprint
from pathlib import Path

_TUPLE_TAG = "__tuple__"


def load_file(path, **kwargs):
    p = str(path)
    if p.endswith((".pkl", ".pickle")):
        with open(p, "rb") as f:
            return pickle.load(f, **kwargs)
    if p.endswith(".json"):
        with open(p) as f:
            return json.load(f, **kwargs)
    if p.endswith((".yaml", ".yml")):
        import yaml

        with open(p) as f:
            return yaml.safe_load(f)
    raise ValueError(f"unknown config format: {p} (use .json, .yaml / .yml or .pkl)")


def save_file(path, data, **kwargs):
    p = str(path)
    if os.path.dirname(p):
        os.makedirs(os.path.dirname(p), exist_ok=True)
    if p.endswith((".pkl", ".pickle")):
        with open(p, "wb") as f:
            pickle.dump(data, f, **kwargs)
    elif p.endswith(".json"):
        kwargs.setdefault("indent", 4)
        with open(p, "w") as f:
            json.dump(data, f, **kwargs)
    elif p.endswith((".yaml", ".yml")):
        import yaml

        with open(p, "w") as f:
            yaml.safe_dump(data, f, **kwargs)
    else:
        raise ValueError(f"unknown config format: {p} (use .json, .yaml / .yml or .pkl)")


class Config(dict):
    def __init__(self, *args, **kwargs):
        super().__init__()
        for k, v in dict(*args, **kwargs).items():
            self[k] = v

    @staticmethod
    def _wrap(v):
        if isinstance(v, dict) and not isinstance(v, Config):
            return Config(v)
        if isinstance(v, list) and v and v[0] == _TUPLE_TAG:      # a tuple that went through JSON
            return tuple(Config._wrap(x) for x in v[1:])
        if isinstance(v, (list, tuple)):
            return type(v)(Config._wrap(x) for x in v)
        return v

    def __setitem__(self, k, v):
        super().__setitem__(k, self._wrap(v))

    def __getattr__(self, k):
        try:
            return self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __setattr__(self, k, v):
        self[k] = v

    def __delattr__(self, k):
        try:
            del self[k]
        except KeyError as e:
            raise AttributeError(k) from e

    def __str__(self):
        return "Config:\n" + self.pretty_text

    @property
    def pretty_text(self) -> str:
        return pprint.pformat(self.to_dict())

    # ---- dict protocol with wrapping -----------------------------------------------------------------
    def update(self, e=None, **f):
        d = dict(e or {})
        d.update(f)
        for k, v in d.items():
            force = False
            if isinstance(v, dict):
                v = dict(v)
                force = bool(v.pop("__force__", False))
            if isinstance(v, dict) and isinstance(self.get(k), Config) and not force:
                self[k].update(v)
            else:
                self[k] = v
        return self

    merge = update

    def setdefault(self, k, d=None):
        if k not in self:
            self[k] = d
        return self[k]

    def copy(self):
        return copy.deepcopy(self)

    def to_dict(self, tuple_as_list: bool = False):
        def un(v):
            if isinstance(v, dict):
                return {k: un(x) for k, x in v.items()}
            if isinstance(v, tuple):
                items = [un(x) for x in v]
                return [_TUPLE_TAG] + items if tuple_as_list else tuple(items)
            if isinstance(v, list):
                return [un(x) for x in v]
            return v

        return un(self)

    # ---- files ---------------------------------------------------------------------------------------
    def save(self, path):
        p = str(path)
        save_file(p, self.to_dict(tuple_as_list=p.endswith((".json", ".yaml", ".yml"))))

    dump = save

    @classmethod
    def load(cls, path):
        p = Path(path)
        if p.suffix not in (".json", ".yaml", ".yml", ".pkl", ".pickle"):
            if p.suffix in (".py", ".config"):
                raise ValueError(f"{p}: python-module configs are not supported; use json / yaml / pickle")
            return cls(pickle.loads(p.read_bytes()))               # suffix-less files written by older dumps
        return cls(load_file(str(p)))

    def merge_from_file(self, path):
        return self.update(Config.load(path))


def load_config(config_or_path) -> Config:
    """A ``Config`` from a file path, a folder containing ``config.json``, a mapping or a ``Config``."""
    if isinstance(config_or_path, Config):
        return config_or_path
    if isinstance(config_or_path, dict):
        return Config(config_or_path)
    if isinstance(config_or_path, (str, os.PathLike)):
        p = str(config_or_path)
        return Config.load(os.path.join(p, "config.json") if os.path.isdir(p) else p)
    raise TypeError(f"cannot build a Config from {type(config_or_path).__name__}")
