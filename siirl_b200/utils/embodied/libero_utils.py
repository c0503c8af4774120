"""Conventions between OpenVLA-style policies and LIBERO / robosuite environments (the reference keeps them in
siirl/utils/embodied/libero_utils.py and inside its adapter, siirl/environment/embodied/adapters/libero.py:313-356):
gripper sign conventions, the no-op action used while the scene settles, the proprioceptive state vector, camera frame
orientation, and saving a rollout as a video file."""
from __future__ import annotations

import math
import os
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

# delta position (3), delta rotation (3), gripper: -1 opens, +1 closes in robosuite
DUMMY_ACTION = [0.0, 0.0, 0.0, 0.0, 0.0, 0.0, -1.0]


def dummy_action(model_family: str = "openvla") -> List[float]:
    """The action that holds the arm still with the gripper open (sent for a few steps after a reset: objects dropped
    into the scene are still falling)."""
    return list(DUMMY_ACTION)


def normalize_gripper_action(action: np.ndarray, binarize: bool = True) -> np.ndarray:
    """Policies are trained on gripper commands in ``[0, 1]``; the simulator wants ``[-1, 1]``.  ``binarize`` snaps to
    the two ends (sign), which is what the data collection did."""
    a = np.array(action, dtype=np.float32, copy=True)
    a[..., -1] = 2.0 * a[..., -1] - 1.0
    if binarize:
        a[..., -1] = np.where(a[..., -1] >= 0.0, 1.0, -1.0)       # sign with 0 -> +1, never 0
    return a


def invert_gripper_action(action: np.ndarray) -> np.ndarray:
    """OpenVLA's training data has 0 = close, 1 = open; robosuite has -1 = open, +1 = close: flip the sign."""
    a = np.array(action, dtype=np.float32, copy=True)
    a[..., -1] *= -1.0
    return a


def policy_action_to_env(action: np.ndarray, model_family: str = "openvla") -> np.ndarray:
    """What the adapter applies to every action of a chunk before stepping the simulator."""
    a = normalize_gripper_action(action, binarize=True)
    return invert_gripper_action(a) if model_family in ("openvla", "openvla-oft", "openvla_oft") else a


def quat2axisangle(quat: Sequence[float]) -> np.ndarray:
    """Unit quaternion ``(x, y, z, w)`` -> axis-angle vector (axis times angle in radians)."""
    x, y, z, w = (float(v) for v in quat)
    w = max(-1.0, min(1.0, w))
    den = math.sqrt(max(1.0 - w * w, 0.0))
    if den < 1e-8:
        return np.zeros(3, dtype=np.float32)
    return (np.array([x, y, z], dtype=np.float32) * (2.0 * math.acos(w) / den)).astype(np.float32)


def camera_frame(obs: Dict[str, Any], key: str) -> Optional[np.ndarray]:
    """robosuite renders upside down and mirrored relative to the training images: rotate by 180 degrees."""
    img = obs.get(key)
    return None if img is None else np.ascontiguousarray(np.asarray(img)[::-1, ::-1])


def proprio_state(obs: Dict[str, Any]) -> Optional[np.ndarray]:
    """End-effector position (3), orientation as axis-angle (3), gripper joint positions (2): the 8 numbers OpenVLA-OFT
    feeds its proprioception projector."""
    if "robot0_eef_pos" not in obs:
        return None
    parts = [np.asarray(obs["robot0_eef_pos"], dtype=np.float32)]
    if "robot0_eef_quat" in obs:
        parts.append(quat2axisangle(obs["robot0_eef_quat"]))
    if "robot0_gripper_qpos" in obs:
        parts.append(np.asarray(obs["robot0_gripper_qpos"], dtype=np.float32))
    return np.concatenate(parts)


def save_rollout_video(frames: Sequence[np.ndarray], out_dir: str, task_name: str, step_idx: int, success: bool,
                       fps: int = 30) -> str:
    """Write one episode's frames (``[H, W, 3] uint8``) under ``out_dir``; returns the path.  Uses ``imageio`` (mp4)
    when it is installed, an animated GIF through Pillow otherwise, and a compressed ``.npz`` when neither is."""
    os.makedirs(out_dir, exist_ok=True)
    safe = "".join(c if c.isalnum() or c in "-_" else "_" for c in task_name.lower())[:60]
    stem = os.path.join(out_dir, f"step={step_idx}--success={bool(success)}--task={safe}")
    frames = [np.asarray(f, dtype=np.uint8) for f in frames]
    try:
        import imageio  # type: ignore
        path = stem + ".mp4"
        with imageio.get_writer(path, fps=fps) as w:
            for f in frames:
                w.append_data(f)
        return path
    except Exception:  # noqa: BLE001
        pass
    try:
        from PIL import Image  # type: ignore
        path = stem + ".gif"
        ims = [Image.fromarray(f) for f in frames]
        ims[0].save(path, save_all=True, append_images=ims[1:], duration=max(1, int(1000 / fps)), loop=0)
        return path
    except Exception:  # noqa: BLE001
        path = stem + ".npz"
        np.savez_compressed(path, frames=np.stack(frames))
        return path
