"""``VideoFolderDataset``: real clips for the encoder ranks, in the item format of ``FakeDataset`` (``prompts``,
``images [T,3,H,W]`` in [-1, 1], ``raw_first_image``, ``index``), so it drops into the same producer loop.

The reference only accepts its random ``FakeDataset`` (teletron/datasets/build.py:30-35); this is the loader a real
run needs.  A data root holds the clips plus one of
  * ``metadata.jsonl`` with one ``{"video": "clips/a.mp4", "caption": "..."}`` object per line,
  * ``metadata.csv`` with ``video,caption`` columns,
  * or a ``<clip>.txt`` caption file beside every video.
Frames are taken with a fixed stride from the start of the clip (the last frame is repeated when the clip is short),
resized so that the target box is covered and centre-cropped; captions pass through ``clean_prompt``.
"""
from __future__ import annotations

import csv
import json
import os
from typing import List, Sequence, Tuple

import torch
from torch.utils.data import Dataset

from ..utils.prompt import clean_prompt
from ..utils.video_io import read_video_frames
from .registry import DATASETS

_VIDEO_EXT = (".mp4", ".avi", ".mov", ".mkv", ".webm")


def _index_root(root: str) -> List[Tuple[str, str]]:
    jl, cs = os.path.join(root, "metadata.jsonl"), os.path.join(root, "metadata.csv")
    items: List[Tuple[str, str]] = []
    if os.path.exists(jl):
        with open(jl) as f:
            for n, line in enumerate(f, 1):
                if not line.strip():
                    continue
                rec = json.loads(line)
                if "video" not in rec:
                    raise ValueError(f"{jl}:{n}: no \"video\" field")
                items.append((os.path.join(root, rec["video"]), str(rec.get("caption", ""))))
    elif os.path.exists(cs):
        with open(cs, newline="") as f:
            for rec in csv.DictReader(f):
                items.append((os.path.join(root, rec["video"]), rec.get("caption", "") or ""))
    else:
        for d, _, files in sorted(os.walk(root)):
            for fn in sorted(files):
                if fn.lower().endswith(_VIDEO_EXT):
                    p = os.path.join(d, fn)
                    txt = os.path.splitext(p)[0] + ".txt"
                    cap = open(txt).read().strip() if os.path.exists(txt) else ""
                    items.append((p, cap))
    return items


def resize_center_crop(frames: torch.Tensor, height: int, width: int) -> torch.Tensor:
    """uint8/float [T,3,H,W] -> float [T,3,height,width]: scale so both sides cover the box, then crop the centre."""
    _, _, H, W = frames.shape
    s = max(height / H, width / W)
    nh, nw = max(int(round(H * s)), height), max(int(round(W * s)), width)
    x = torch.nn.functional.interpolate(frames.float(), size=(nh, nw), mode="bilinear", align_corners=False,
                                        antialias=s < 1.0)
    top, left = (nh - height) // 2, (nw - width) // 2
    return x[:, :, top:top + height, left:left + width]


@DATASETS.register("VideoFolderDataset")
class VideoFolderDataset(Dataset):
    def __init__(self, data_path, num_frames=81, height=480, width=832, frame_stride=1, clean_captions=True,
                 backend=None, seed=0, min_length=0, **_):
        """``min_length``: the sample count the run will ask for; the clip list is repeated (whole epochs) until it
        covers it, because the resumable samplers walk ``range(len(dataset))`` once."""
        roots: Sequence[str] = [data_path] if isinstance(data_path, str) else list(data_path or [])
        if not roots:
            raise ValueError("VideoFolderDataset needs --data-path <folder> [<folder> ...]")
        self.items: List[Tuple[str, str]] = []
        for r in roots:
            if not os.path.isdir(r):
                raise FileNotFoundError(f"data path {r} is not a folder")
            self.items += _index_root(r)
        if not self.items:
            raise ValueError(f"no videos found under {roots}")
        self.num_frames, self.height, self.width = num_frames, height, width
        self.stride, self.clean, self.backend = max(int(frame_stride), 1), clean_captions, backend
        self.min_length = min_length

    def __len__(self):
        n = len(self.items)
        return n * max(1, -(-int(self.min_length) // n))

    def __getitem__(self, idx):
        path, caption = self.items[int(idx) % len(self.items)]
        fr = read_video_frames(path, num_frames=self.num_frames, stride=self.stride, backend=self.backend)  # [T,H,W,3]
        x = fr.permute(0, 3, 1, 2)
        if x.shape[0] < self.num_frames:                     # short clip: hold the last frame
            x = torch.cat([x, x[-1:].expand(self.num_frames - x.shape[0], -1, -1, -1)], dim=0)
        x = resize_center_crop(x, self.height, self.width) / 127.5 - 1.0
        return dict(prompts=clean_prompt(caption) if self.clean else caption, images=x,
                    raw_first_image=x[0].clone(), index=int(idx))
