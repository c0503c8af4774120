"""Image and video fetching for vision-language datasets (reference: siirl/data_coordinator/dataloader/vision_utils.py,
which delegates to ``qwen_vl_utils.fetch_image / fetch_video``; that package is not available offline, so the rules
are restated here).

``process_image`` accepts a PIL image, an array / tensor, ``{"bytes": ...}``, ``{"image": <path | PIL | array>}`` and
returns an RGB ``[3, H, W]`` float tensor in [0, 1] resized so that both sides are multiples of 28 and the area lies in
``[min_pixels, max_pixels]``.

``process_video`` accepts ``{"video": <list of frames | path to .npy / .pt | path to a video file>, ...}`` with the
Qwen2-VL sampling keys (``nframes`` or ``fps`` with ``min_frames`` / ``max_frames``) and returns ``[n_frames, 3, H, W]``
(n_frames a multiple of 2).  Video files are decoded with OpenCV when it is installed.
"""
from __future__ import annotations

import math
import os
from typing import Any, List, Optional

import numpy as np
import torch
import torch.nn.functional as F

IMAGE_FACTOR = 28
FRAME_FACTOR = 2
FPS = 2.0
FPS_MIN_FRAMES = 4
FPS_MAX_FRAMES = 768
VIDEO_MIN_PIXELS = 128 * 28 * 28
VIDEO_MAX_PIXELS = 768 * 28 * 28


def _round(x: float, f: int) -> int:
    return max(f, int(round(x / f)) * f)


def smart_resize(h: int, w: int, factor: int = IMAGE_FACTOR, min_pixels: int = 4 * 28 * 28,
                 max_pixels: int = 16384 * 28 * 28):
    if max(h, w) / max(min(h, w), 1) > 200:
        raise ValueError(f"aspect ratio of a {h}x{w} image is beyond 200")
    hb, wb = _round(h, factor), _round(w, factor)
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb, wb = max(factor, math.floor(h / beta / factor) * factor), max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb, wb = math.ceil(h * beta / factor) * factor, math.ceil(w * beta / factor) * factor
    return hb, wb


def _load_rgb(src: Any) -> torch.Tensor:
    """-> ``[3, H, W]`` float in [0, 1]."""
    if isinstance(src, dict):
        if "bytes" in src:
            import io

            from PIL import Image
            src = Image.open(io.BytesIO(src["bytes"]))
        else:
            src = src.get("image", src.get("path"))
    if isinstance(src, str):
        from PIL import Image
        src = Image.open(src[7:] if src.startswith("file://") else src)
    if hasattr(src, "convert"):
        src = np.asarray(src.convert("RGB"))
    t = src if isinstance(src, torch.Tensor) else torch.as_tensor(np.asarray(src))
    if t.dim() == 3 and t.shape[-1] == 3 and t.shape[0] != 3:
        t = t.permute(2, 0, 1)
    t = t.float()
    return t / 255.0 if t.max() > 1.5 else t


def process_image(image: Any, max_pixels: int, min_pixels: int) -> torch.Tensor:
    x = _load_rgb(image)
    h2, w2 = smart_resize(x.shape[1], x.shape[2], IMAGE_FACTOR, min_pixels, max_pixels)
    if (h2, w2) != tuple(x.shape[1:]):
        x = F.interpolate(x[None], size=(h2, w2), mode="bilinear", align_corners=False, antialias=True)[0]
    return x.clamp(0, 1)


def sample_frame_indices(total: int, video_fps: float, nframes: Optional[int] = None, fps: Optional[float] = None,
                         min_frames: int = FPS_MIN_FRAMES, max_frames: int = FPS_MAX_FRAMES) -> List[int]:
    """Evenly spaced frame indices: ``nframes`` of them, or as many as ``fps`` asks for over the clip's duration
    (clamped to ``[min_frames, max_frames]``), rounded to a multiple of 2 and never more than ``total``."""
    if nframes is not None and fps is not None:
        raise ValueError("give either nframes or fps, not both")
    if nframes is not None:
        n = _round(nframes, FRAME_FACTOR)
    else:
        fps = FPS if fps is None else fps
        lo = math.ceil(min_frames / FRAME_FACTOR) * FRAME_FACTOR
        hi = math.floor(min(max_frames, total) / FRAME_FACTOR) * FRAME_FACTOR
        n = total / max(video_fps, 1e-6) * fps
        n = min(max(n, lo), max(hi, FRAME_FACTOR))
        n = math.floor(n / FRAME_FACTOR) * FRAME_FACTOR
    n = max(FRAME_FACTOR, min(int(n), max(total // FRAME_FACTOR * FRAME_FACTOR, FRAME_FACTOR)))
    return [int(round(i)) for i in np.linspace(0, max(total - 1, 0), n)]


def _decode_video_file(path: str):
    ext = os.path.splitext(path)[1].lower()
    if ext == ".npy":
        return torch.as_tensor(np.load(path)), FPS
    if ext in (".pt", ".pth"):
        return torch.load(path, map_location="cpu"), FPS
    try:
        import cv2
    except ImportError as e:  # pragma: no cover
        raise RuntimeError(f"decoding {path} needs OpenCV (cv2); pass frames, a .npy or a .pt tensor instead") from e
    cap = cv2.VideoCapture(path)
    if not cap.isOpened():
        raise FileNotFoundError(path)
    fps = cap.get(cv2.CAP_PROP_FPS) or FPS
    frames = []
    while True:
        ok, frame = cap.read()
        if not ok:
            break
        frames.append(torch.from_numpy(cv2.cvtColor(frame, cv2.COLOR_BGR2RGB)))
    cap.release()
    if not frames:
        raise ValueError(f"{path}: no frames decoded")
    return torch.stack(frames), float(fps)


def process_video(video: dict, nframes: Optional[int] = None, fps: Optional[float] = None,
                  fps_min_frames: Optional[int] = None, fps_max_frames: Optional[int] = None,
                  max_pixels: Optional[int] = None, min_pixels: Optional[int] = None) -> torch.Tensor:
    """Video dict -> ``[n_frames, 3, H, W]`` float tensor in [0, 1]."""
    if not isinstance(video, dict) or "video" not in video:
        raise NotImplementedError('a video is {"type": "video", "video": <frames | path>, optional "fps" / "nframes" '
                                  '/ "min_frames" / "max_frames" / "min_pixels" / "max_pixels"}')
    if nframes is not None and fps is not None:
        raise ValueError("give either nframes or fps, not both")
    v = dict(video)
    if "nframes" not in v and "fps" not in v:
        if nframes is not None:
            v["nframes"] = nframes
        elif fps is not None:
            v["fps"] = fps
            if fps_min_frames is not None:
                v["min_frames"] = fps_min_frames
            if fps_max_frames is not None:
                v["max_frames"] = fps_max_frames
    src = v["video"]
    if isinstance(src, (list, tuple)):              # a list of frames: every frame is kept unless sampling is asked for
        frames = torch.stack([_load_rgb(f) for f in src])
        video_fps = float(v.get("sample_fps", FPS))
        explicit = "nframes" in v or "fps" in v
    else:
        raw, video_fps = (src, float(v.get("sample_fps", FPS))) if isinstance(src, (torch.Tensor, np.ndarray)) else \
            _decode_video_file(src[7:] if isinstance(src, str) and src.startswith("file://") else src)
        raw = torch.as_tensor(raw)
        if raw.dim() == 4 and raw.shape[-1] == 3 and raw.shape[1] != 3:
            raw = raw.permute(0, 3, 1, 2)
        frames = raw.float()
        frames = frames / 255.0 if frames.max() > 1.5 else frames
        explicit = True
    total = frames.shape[0]
    if explicit:
        idx = sample_frame_indices(total, video_fps, v.get("nframes"), v.get("fps") if "nframes" not in v else None,
                                   int(v.get("min_frames", FPS_MIN_FRAMES)), int(v.get("max_frames", FPS_MAX_FRAMES)))
        frames = frames[torch.tensor(idx)]
    if frames.shape[0] % FRAME_FACTOR:
        frames = torch.cat([frames, frames[-1:]])
    n, _, h, w = frames.shape
    lo = int(v.get("min_pixels", min_pixels or VIDEO_MIN_PIXELS))
    total_pixels = int(v.get("total_pixels", 24576 * 28 * 28))
    hi = max(min(int(v.get("max_pixels", max_pixels or VIDEO_MAX_PIXELS)), total_pixels // n * FRAME_FACTOR),
             int(lo * 1.05))
    h2, w2 = smart_resize(h, w, IMAGE_FACTOR, lo, hi)
    if (h2, w2) != (h, w):
        frames = F.interpolate(frames, size=(h2, w2), mode="bilinear", align_corners=False, antialias=True)
    return frames.clamp(0, 1)
