"""Attribute-style configuration dictionary with json / yaml / pickle IO
(teletron/train/config.py:69-172)."""
from __future__ import annotations

import json
import pickle
from pathlib import Path


class Config(dict):
    def __init__(self, *args, **kwargs):
        super().__init__()
        for k, v in dict(*args, **kwargs).items():
            self[k] = v

    @staticmethod
    def _wrap(v):
        if isinstance(v, dict) and not isinstance(v, Config):
            return Config(v)
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
        del self[k]

    def to_dict(self):
        def un(v):
            if isinstance(v, Config):
                return {k: un(x) for k, x in v.items()}
            if isinstance(v, (list, tuple)):
                return type(v)(un(x) for x in v)
            return v

        return un(self)

    def merge(self, other):
        for k, v in dict(other).items():
            if isinstance(v, dict) and isinstance(self.get(k), Config):
                self[k].merge(v)
            else:
                self[k] = v
        return self

    def dump(self, path):
        p = Path(path)
        if p.suffix == ".json":
            p.write_text(json.dumps(self.to_dict(), indent=2))
        elif p.suffix in (".yaml", ".yml"):
            import yaml

            p.write_text(yaml.safe_dump(self.to_dict()))
        else:
            p.write_bytes(pickle.dumps(self.to_dict()))

    @classmethod
    def load(cls, path):
        p = Path(path)
        if p.suffix == ".json":
            return cls(json.loads(p.read_text()))
        if p.suffix in (".yaml", ".yml"):
            import yaml

            return cls(yaml.safe_load(p.read_text()))
        return cls(pickle.loads(p.read_bytes()))
