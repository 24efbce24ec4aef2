"""Dataset registry and ``build_dataset`` (teletron/datasets/registry.py:17-63, build.py:30-35)."""
from __future__ import annotations

from ..models.registry import Registry

DATASETS = Registry("dataset")


def build_dataset(name_or_spec, **kwargs):
    """``build_dataset("FakeDataset", num_frames=...)`` or ``build_dataset({"type": "FakeDataset", ...})``."""
    return DATASETS.build(name_or_spec, **kwargs)
