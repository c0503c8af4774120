"""Headless synthetic manipulation environment.

The reference's embodied path drives LIBERO / robosuite / MuJoCo with off-screen GL cameras
(siirl/environment/embodied/adapters/libero.py:205-311).  That needs a graphics stack; this environment keeps the
same interface and data shapes without one: a planar reach task (gripper position, goal position, open/close state),
7-dimensional continuous actions like a robot arm's delta pose + gripper, 256x256x3 camera observations rendered
by the CUDA rasteriser of ``siirl_b200.ops.image`` (numpy twin on CPU), success when the gripper is within 5 % of the
goal.  Tasks are seeded goal/start layouts, so ``task_ids`` / ``trial_ids`` select reproducible episodes."""
from __future__ import annotations

from typing import Any, Dict, List, Optional

import numpy as np
import torch

from ...ops.image import raster_synth_env
from .base import BaseVLAEnvironment


class SyntheticReachEnv(BaseVLAEnvironment):
    def __init__(self, num_envs: int = 16, max_steps: int = 64, image_size: int = 256, device: str = "cpu",
                 success_radius: float = 0.05, action_scale: float = 0.08, num_tasks: int = 10):
        self.num_envs = num_envs
        self.max_steps = max_steps
        self.image_size = image_size
        self.device = torch.device(device)
        self.success_radius = success_radius
        self.action_scale = action_scale
        self.num_tasks = num_tasks
        self.state = np.zeros((num_envs, 8), dtype=np.float32)
        self.steps = np.zeros(num_envs, dtype=np.int64)
        self.done = np.ones(num_envs, dtype=bool)
        self.success = np.zeros(num_envs, dtype=bool)
        self.task_ids = np.zeros(num_envs, dtype=np.int64)

    def task_description(self, task_id: int) -> str:
        return f"move the gripper to the green target (layout {task_id % self.num_tasks})"

    def _render(self) -> torch.Tensor:
        st = torch.from_numpy(self.state).to(self.device)
        return raster_synth_env(st, self.image_size, self.image_size)

    def _wrist_view(self, img: torch.Tensor) -> torch.Tensor:
        """A second camera: the quarter of the scene around the gripper, magnified to the full frame (what a wrist
        camera sees: the surroundings of the end effector)."""
        S = self.image_size
        half = S // 4
        cx = np.clip((self.state[:, 0] * S).astype(np.int64), half, S - half)
        cy = np.clip((self.state[:, 1] * S).astype(np.int64), half, S - half)
        dev = img.device
        zoom = torch.arange(S, device=dev) // 2                                  # every source pixel twice
        rows = torch.from_numpy(cy - half).to(dev)[:, None] + zoom[None, :]      # [N, S]
        cols = torch.from_numpy(cx - half).to(dev)[:, None] + zoom[None, :]
        n = torch.arange(self.num_envs, device=dev)[:, None, None]
        return img[n, rows[:, :, None], cols[:, None, :]]

    def _obs(self) -> List[Dict[str, Any]]:
        img = self._render()
        wrist = self._wrist_view(img)
        return [{"image": img[i], "wrist_image": wrist[i], "state": self.state[i, :5].copy(), "task_description": self.task_description(
            int(self.task_ids[i])), "step": int(self.steps[i]), "done": bool(self.done[i]),
            "success": bool(self.success[i])} for i in range(self.num_envs)]

    async def reset(self, task_ids: Optional[List[int]] = None, trial_ids: Optional[List[int]] = None):
        task_ids = list(task_ids) if task_ids is not None else list(range(self.num_envs))
        trial_ids = list(trial_ids) if trial_ids is not None else [0] * self.num_envs
        for i in range(self.num_envs):
            rng = np.random.RandomState(1000 * (task_ids[i] % self.num_tasks) + trial_ids[i])
            goal = rng.uniform(0.15, 0.85, 2)
            start = rng.uniform(0.15, 0.85, 2)
            while np.linalg.norm(goal - start) < 0.25:
                start = rng.uniform(0.15, 0.85, 2)
            self.state[i] = [start[0], start[1], goal[0], goal[1], 1.0, 0, 0, 0]
            self.task_ids[i] = task_ids[i]
        self.steps[:] = 0
        self.done[:] = False
        self.success[:] = False
        return self._obs()

    async def step(self, action) -> List[Dict[str, Any]]:
        """``action [num_envs, 7]`` or a chunk ``[num_envs, chunk, 7]`` in [-1, 1]."""
        a = np.asarray(action, dtype=np.float32)
        if a.ndim == 2:
            a = a[:, None, :]
        rewards = np.zeros(self.num_envs, dtype=np.float32)
        for c in range(a.shape[1]):
            live = ~self.done
            delta = np.clip(a[:, c, :2], -1, 1) * self.action_scale
            self.state[live, :2] = np.clip(self.state[live, :2] + delta[live], 0.0, 1.0)
            self.state[live, 4] = (a[live, c, 6] > 0).astype(np.float32)
            self.steps[live] += 1
            dist = np.linalg.norm(self.state[:, :2] - self.state[:, 2:4], axis=1)
            hit = live & (dist < self.success_radius)
            self.success |= hit
            rewards += hit.astype(np.float32)
            self.done |= hit | (self.steps >= self.max_steps)
        obs = self._obs()
        for i, o in enumerate(obs):
            o["reward"] = float(rewards[i])
        return obs
