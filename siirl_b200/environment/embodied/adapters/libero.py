"""LIBERO adapter (interface of siirl/environment/embodied/adapters/libero.py:38-356).

LIBERO renders camera observations with robosuite's ``OffScreenRenderEnv`` (MuJoCo + off-screen OpenGL).  Machines
without a graphics stack cannot create that renderer; the adapter then raises ``EnvironmentUnavailable`` with the
reason, and ``make_environment("synthetic")`` provides the headless stand-in with the same method signatures."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import numpy as np

from ..base import BaseVLAEnvironment
from ..venv import SubprocVectorEnv


class EnvironmentUnavailable(RuntimeError):
    pass


class LIBEROAdapter(BaseVLAEnvironment):
    def __init__(self, env_name: str = "libero_10", num_envs: int = 16, max_steps: int = 512, num_steps_wait: int = 10,
                 model_family: str = "openvla", gpu_ids: Optional[List[int]] = None, **kwargs):
        try:
            from libero.libero import benchmark  # type: ignore
            from libero.libero.envs import OffScreenRenderEnv  # type: ignore  # noqa: F401
        except Exception as e:  # noqa: BLE001
            raise EnvironmentUnavailable(
                "LIBERO / robosuite (MuJoCo off-screen rendering) is not available on this machine: "
                f"{type(e).__name__}: {e}.  Use env_type=synthetic for the headless environment.") from e
        self.benchmark = benchmark.get_benchmark_dict()[env_name]()
        self.num_envs, self.max_steps, self.num_steps_wait = num_envs, max_steps, num_steps_wait
        self.model_family = model_family
        self.gpu_ids = gpu_ids or [0]
        self.env = None
        self.steps = np.zeros(num_envs, dtype=np.int64)

    def _make_fns(self, task_ids: List[int]):
        import os
        from libero.libero import get_libero_path  # type: ignore
        from libero.libero.envs import OffScreenRenderEnv  # type: ignore
        fns = []
        for k, tid in enumerate(task_ids):
            task = self.benchmark.get_task(tid)
            bddl = os.path.join(get_libero_path("bddl_files"), task.problem_folder, task.bddl_file)
            gpu = self.gpu_ids[k % len(self.gpu_ids)]
            fns.append(lambda b=bddl, g=gpu: OffScreenRenderEnv(bddl_file_name=b, camera_heights=256,
                                                                camera_widths=256, render_gpu_device_id=g))
        return fns

    async def reset(self, task_ids=None, trial_ids=None) -> List[Dict[str, Any]]:
        task_ids = list(task_ids or range(self.num_envs))
        if self.env is not None:
            self.env.close()
        self.env = SubprocVectorEnv(self._make_fns(task_ids))
        obs = self.env.reset()
        self.steps[:] = 0
        return [{"image": o["agentview_image"][::-1, ::-1], "wrist_image": self._wrist(o), "state": o.get("robot0_eef_pos"),
                 "task_description": self.benchmark.get_task(t).language, "step": 0, "done": False, "success": False}
                for o, t in zip(obs, task_ids)]

    async def step(self, action) -> List[Dict[str, Any]]:
        obs, rew, done, info = self.env.step(np.asarray(action))
        self.steps += 1
        return [{"image": o["agentview_image"][::-1, ::-1], "wrist_image": self._wrist(o), "reward": float(r),
                 "done": bool(d) or self.steps[i] >=
                 self.max_steps, "success": bool(d), "step": int(self.steps[i])}
                for i, (o, r, d) in enumerate(zip(obs, rew, done))]

    @staticmethod
    def _wrist(o):
        """Wrist-camera frame (rotated like the third-person view), ``None`` when the suite renders none."""
        w = o.get("robot0_eye_in_hand_image")
        return w[::-1, ::-1] if w is not None else None

    def close(self) -> None:
        if self.env is not None:
            self.env.close()
