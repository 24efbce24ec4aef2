"""Headless video reading / writing helpers.

Covers what the reference spreads over two modules (teletron/utils/video_utils.py:12-65: ``load_video``,
``save_video``, ``get_fps``, ``sample_video``, ``add_music_to_video``; teletron/utils/read_video.py:21-268:
``read_video`` with a PyAV and an OpenCV backend, time-window selection in seconds, ``TCHW`` / ``THWC``
output and a ``video_fps`` info dict).  Backends are probed at call time in the order PyAV, decord, imageio,
OpenCV, so the module imports without any of them; the window-system calls of the reference's OpenCV reader
are not carried over, and the audio copy runs ffmpeg with an argument list instead of a shell string.
"""
from __future__ import annotations

import os
import shutil
import subprocess
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

import numpy as np
import torch


# --------------------------------------------------------------------------------- decoding
def _frames_av(path: str) -> Tuple[Iterator[np.ndarray], float]:
    import av

    container = av.open(path)
    stream = container.streams.video[0]
    fps = float(stream.average_rate) if stream.average_rate else 0.0

    def gen():
        try:
            for fr in container.decode(video=0):
                yield fr.to_ndarray(format="rgb24")
        finally:
            container.close()          # PyAV leaks decoder threads when containers are left open

    return gen(), fps


def _frames_decord(path: str) -> Tuple[Iterator[np.ndarray], float]:
    from decord import VideoReader

    vr = VideoReader(path)
    fps = float(vr.get_avg_fps())

    def gen():
        for i in range(len(vr)):
            fr = vr[i]
            yield fr.numpy() if isinstance(fr, torch.Tensor) else fr.asnumpy()

    return gen(), fps


def _frames_imageio(path: str) -> Tuple[Iterator[np.ndarray], float]:
    import imageio.v3 as iio

    try:
        fps = float(iio.immeta(path).get("fps", 0.0))
    except Exception:
        fps = 0.0
    return (np.asarray(fr)[..., :3] for fr in iio.imiter(path)), fps


def _frames_cv2(path: str) -> Tuple[Iterator[np.ndarray], float]:
    import cv2

    cap = cv2.VideoCapture(path)
    if not cap.isOpened():
        raise ValueError(f"cannot open video {path}")
    fps = float(cap.get(cv2.CAP_PROP_FPS) or 0.0)

    def gen():
        try:
            while True:
                ok, fr = cap.read()
                if not ok:
                    break
                yield fr[:, :, ::-1]   # BGR -> RGB
        finally:
            cap.release()

    return gen(), fps


_BACKENDS = {"av": _frames_av, "decord": _frames_decord, "imageio": _frames_imageio, "cv2": _frames_cv2}


def open_frames(path: str, backend: Optional[str] = None) -> Tuple[Iterator[np.ndarray], float, str]:
    """(iterator of RGB uint8 [H,W,3] frames, average fps, backend name).  ``backend=None`` takes the
    first installed one."""
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    names = [backend] if backend else list(_BACKENDS)
    last: Optional[Exception] = None
    for n in names:
        if n not in _BACKENDS:
            raise ValueError(f"unknown video backend {n!r} (choose from {sorted(_BACKENDS)})")
        try:
            it, fps = _BACKENDS[n](path)
            return it, fps, n
        except ImportError as e:
            last = e
    raise RuntimeError(f"no video backend available for {path}: {last}")


def read_video_frames(path: str, num_frames: Optional[int] = None, stride: int = 1, start: int = 0,
                      backend: Optional[str] = None) -> torch.Tensor:
    """uint8 [T, H, W, 3] (RGB): every ``stride``-th frame from frame ``start``, at most ``num_frames``."""
    it, _, _ = open_frames(path, backend)
    frames: List[np.ndarray] = []
    for i, fr in enumerate(it):
        if i >= start and (i - start) % stride == 0:
            frames.append(np.ascontiguousarray(fr))
            if num_frames and len(frames) >= num_frames:
                break
    if hasattr(it, "close"):
        it.close()
    if not frames:
        raise RuntimeError(f"no frames decoded from {path}")
    return torch.from_numpy(np.stack(frames))


def read_video(video_path: str, backend: Optional[str] = "av", start_sec: float = 0.0,
               end_sec: Optional[float] = None, output_format: str = "TCHW") -> Tuple[torch.Tensor, Dict]:
    """(frames, {"video_fps": fps}) like the reference's ``read_video`` (read_video.py:258-268): uint8
    ``[T,3,H,W]`` (or ``[T,H,W,3]`` with ``output_format="THWC"``), optionally only the frames whose
    presentation time lies in ``[start_sec, end_sec]``.  A missing PyAV falls back to the next backend."""
    output_format = output_format.upper()
    if output_format not in ("THWC", "TCHW"):
        raise ValueError(f"output_format should be either 'THWC' or 'TCHW', got {output_format}.")
    if end_sec is not None and end_sec < start_sec:
        raise ValueError(f"end_sec ({end_sec}) is before start_sec ({start_sec})")
    try:
        it, fps, _ = open_frames(video_path, backend)
    except RuntimeError:
        it, fps, _ = open_frames(video_path, None)
    frames = []
    for i, fr in enumerate(it):
        t = i / fps if fps > 0 else 0.0
        if t < start_sec:
            continue
        if end_sec is not None and t > end_sec:
            break
        frames.append(np.ascontiguousarray(fr))
    if hasattr(it, "close"):
        it.close()
    if frames:
        out = torch.from_numpy(np.stack(frames))
    else:
        out = torch.empty((0, 1, 1, 3), dtype=torch.uint8)
    if output_format == "TCHW":
        out = out.permute(0, 3, 1, 2)
    return out, {"video_fps": fps}


def load_video(video_path: str) -> List:
    """Every frame as a PIL image (numpy arrays when Pillow is missing)."""
    arr = read_video_frames(video_path).numpy()
    try:
        from PIL import Image

        return [Image.fromarray(a) for a in arr]
    except ImportError:
        return list(arr)


def get_fps(video_path: str) -> float:
    it, fps, _ = open_frames(video_path)
    if hasattr(it, "close"):
        it.close()
    return fps


def sample_video(video, indexes: Sequence[int]) -> np.ndarray:
    """Frames ``indexes`` of ``video`` as one uint8 array [len(indexes), H, W, 3].  ``video`` is a path, a
    decord-style reader (``get_batch``), or anything indexable by frame (tensor, array, list)."""
    idx = np.asarray(indexes, dtype=int)
    if isinstance(video, str):
        n = int(idx.max()) + 1 if idx.size else 0
        return read_video_frames(video, num_frames=n).numpy()[idx]
    if hasattr(video, "get_batch"):
        fr = video.get_batch(np.arange(int(idx.max()) + 1, dtype=int))   # sequential decode, then pick
        fr = fr.numpy() if isinstance(fr, torch.Tensor) else fr.asnumpy()
        return fr[idx]
    if isinstance(video, torch.Tensor):
        return video[torch.as_tensor(idx)].numpy()
    return np.stack([np.asarray(video[int(i)]) for i in idx])


def frames_to_tensor(frames: torch.Tensor) -> torch.Tensor:
    """uint8 [T,H,W,3] -> float [T,3,H,W] in [-1, 1]."""
    return frames.permute(0, 3, 1, 2).float() / 127.5 - 1.0


# --------------------------------------------------------------------------------- encoding
def save_video(frames, path: str, fps: int = 16, **kwargs):
    """frames: list of PIL images / uint8 arrays [H,W,3].  imageio when installed (as the reference),
    else OpenCV's writer (``fourcc`` keyword, default mp4v; MJPG for .avi)."""
    arrs = [np.asarray(f) for f in frames]
    try:
        import imageio

        imageio.mimsave(path, arrs, fps=fps, **kwargs)
        return
    except ImportError:
        pass
    import cv2

    h, w = arrs[0].shape[:2]
    fourcc = kwargs.get("fourcc") or ("MJPG" if path.lower().endswith(".avi") else "mp4v")
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*fourcc), fps, (w, h))
    if not wr.isOpened():
        raise RuntimeError(f"OpenCV cannot open a {fourcc} writer for {path}")
    for a in arrs:
        wr.write(np.ascontiguousarray(a[:, :, ::-1]))
    wr.release()


def add_music_to_video(src_video_path: str, dst_video_path: str, save_video_path: Optional[str] = None) -> str:
    """Copy the audio track of ``src`` onto the (silent) ``dst`` video with ffmpeg, without re-encoding
    (video_utils.py:49-65).  Returns the path written."""
    ffmpeg = shutil.which("ffmpeg")
    if ffmpeg is None:
        raise RuntimeError("ffmpeg is not installed")
    root, ext = os.path.splitext(dst_video_path)
    save_video_path = save_video_path or f"{root}_music{ext}"
    aud_path = os.path.splitext(src_video_path)[0] + ".m4a"
    if os.path.exists(save_video_path):
        os.remove(save_video_path)
    try:
        subprocess.run([ffmpeg, "-i", src_video_path, "-vn", "-y", "-acodec", "copy", aud_path], check=True,
                       capture_output=True)
        subprocess.run([ffmpeg, "-i", dst_video_path, "-i", aud_path, "-vcodec", "copy", "-acodec", "copy",
                        save_video_path], check=True, capture_output=True)
    finally:
        if os.path.exists(aud_path):
            os.remove(aud_path)
    return save_video_path
