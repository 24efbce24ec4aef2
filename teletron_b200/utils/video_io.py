"""Headless video reading / writing helpers (teletron/utils/video_utils.py:12-65,
teletron/utils/read_video.py:21-268).  Backends are probed at call time: PyAV, imageio, OpenCV;
window-system calls of the reference reader are not carried over."""
from __future__ import annotations

from typing import List

import numpy as np
import torch


def read_video_frames(path: str, num_frames: int = None, stride: int = 1, start: int = 0) -> torch.Tensor:
    """Returns uint8 [T, H, W, 3] (RGB)."""
    frames: List[np.ndarray] = []
    try:
        import av

        with av.open(path) as c:
            for i, fr in enumerate(c.decode(video=0)):
                if i >= start and (i - start) % stride == 0:
                    frames.append(fr.to_ndarray(format="rgb24"))
                    if num_frames and len(frames) >= num_frames:
                        break
    except ImportError:
        try:
            import imageio.v3 as iio

            for i, fr in enumerate(iio.imiter(path)):
                if i >= start and (i - start) % stride == 0:
                    frames.append(np.asarray(fr)[..., :3])
                    if num_frames and len(frames) >= num_frames:
                        break
        except ImportError:
            import cv2

            cap = cv2.VideoCapture(path)
            i = 0
            while True:
                ok, fr = cap.read()
                if not ok:
                    break
                if i >= start and (i - start) % stride == 0:
                    frames.append(cv2.cvtColor(fr, cv2.COLOR_BGR2RGB))
                    if num_frames and len(frames) >= num_frames:
                        break
                i += 1
            cap.release()
    if not frames:
        raise RuntimeError(f"no frames decoded from {path}")
    return torch.from_numpy(np.stack(frames))


def frames_to_tensor(frames: torch.Tensor) -> torch.Tensor:
    """uint8 [T,H,W,3] -> float [T,3,H,W] in [-1, 1]."""
    return frames.permute(0, 3, 1, 2).float() / 127.5 - 1.0


def save_video(frames, path: str, fps: int = 16):
    """frames: list of PIL images / uint8 arrays [H,W,3]. Uses OpenCV's writer (mp4v)."""
    import cv2

    arrs = [np.asarray(f) for f in frames]
    h, w = arrs[0].shape[:2]
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), fps, (w, h))
    for a in arrs:
        wr.write(cv2.cvtColor(a, cv2.COLOR_RGB2BGR))
    wr.release()
