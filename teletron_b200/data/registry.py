"""Dataset registry and ``build_dataset`` (teletron/datasets/registry.py:17-63, build.py:30-35)."""
from __future__ import annotations

from ..models.registry import Registry

DATASETS = Registry("dataset")


def build_dataset(name: str, **kwargs):
    return DATASETS.get(name)(**kwargs)
