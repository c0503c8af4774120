"""LIBERO adapter (interface of siirl/environment/embodied/adapters/libero.py:38-356).

LIBERO renders camera observations with robosuite's ``OffScreenRenderEnv`` (MuJoCo + off-screen OpenGL).  Machines
without a graphics stack cannot create that renderer; the adapter then raises ``EnvironmentUnavailable`` with the
reason, and ``make_environment("synthetic")`` provides the headless stand-in with the same method signatures.

Behaviour, per environment slot:

* ``reset(task_ids, trial_ids)``: one simulator per slot for the slot's task (kept while the task list is unchanged),
  initial state ``trial_id`` of the suite's recorded initial states, then ``num_steps_wait`` no-op actions while the
  scene settles.
* ``step(actions)``: ``[N, 7]`` or a chunk ``[N, chunk, 7]``; every action goes through the policy -> simulator gripper
  convention; slots that finished (task solved or ``max_steps`` reached) are not stepped again, inside a chunk or
  after it.
* observations: ``image`` (third-person view), ``wrist_image``, ``state`` (end-effector position, axis-angle
  orientation, gripper joints), ``task_description``, ``step``, ``done``, ``success``.
"""
from __future__ import annotations

import os
from typing import Any, Dict, List, Optional

import numpy as np

from ....utils.embodied import libero_utils as LU
from ..base import BaseVLAEnvironment
from ..venv import DummyVectorEnv, SubprocVectorEnv


class EnvironmentUnavailable(RuntimeError):
    pass


class _SimulatorFactory:
    """Picklable constructor of one simulator (worker processes are spawned, so a closure would not travel)."""

    def __init__(self, bddl_file: str, gpu: int, resolution: int):
        self.bddl_file, self.gpu, self.resolution = bddl_file, gpu, resolution

    def __call__(self):
        from libero.libero.envs import OffScreenRenderEnv  # type: ignore
        return OffScreenRenderEnv(bddl_file_name=self.bddl_file, camera_heights=self.resolution,
                                  camera_widths=self.resolution, render_gpu_device_id=self.gpu)


class LIBEROAdapter(BaseVLAEnvironment):
    def __init__(self, env_name: str = "libero_10", num_envs: int = 16, max_steps: int = 512, num_steps_wait: int = 10,
                 model_family: str = "openvla", gpu_ids: Optional[List[int]] = None, resolution: int = 256,
                 vector_env: str = "subproc", **_unused):
        try:
            from libero.libero import benchmark  # type: ignore
            from libero.libero.envs import OffScreenRenderEnv  # type: ignore  # noqa: F401
        except Exception as e:  # noqa: BLE001
            raise EnvironmentUnavailable(
                "LIBERO / robosuite (MuJoCo off-screen rendering) is not available on this machine: "
                f"{type(e).__name__}: {e}.  Use env_type=synthetic for the headless environment.") from e
        suites = benchmark.get_benchmark_dict()
        if env_name not in suites:
            raise ValueError(f"unknown LIBERO suite '{env_name}' (have: {sorted(suites)})")
        self.benchmark = suites[env_name]()
        self.num_envs, self.max_steps, self.num_steps_wait = num_envs, max_steps, num_steps_wait
        self.model_family = model_family
        self.gpu_ids = gpu_ids or [0]
        self.resolution = resolution
        self.vector_env = vector_env
        self.env = None
        self._env_tasks: Optional[List[int]] = None
        self.task_ids: List[int] = []
        self.steps = np.zeros(num_envs, dtype=np.int64)
        self.done = np.ones(num_envs, dtype=bool)
        self.success = np.zeros(num_envs, dtype=bool)
        self._last: List[Dict[str, Any]] = []

    # ---- construction ----------------------------------------------------------------------------------------------
    def _factories(self, task_ids: List[int]):
        from libero.libero import get_libero_path  # type: ignore
        fns = []
        for k, tid in enumerate(task_ids):
            task = self.benchmark.get_task(tid)
            bddl = os.path.join(get_libero_path("bddl_files"), task.problem_folder, task.bddl_file)
            fns.append(_SimulatorFactory(bddl, self.gpu_ids[k % len(self.gpu_ids)], self.resolution))
        return fns

    def _ensure_envs(self, task_ids: List[int]) -> None:
        if self.env is not None and self._env_tasks == task_ids:
            return
        if self.env is not None:
            self.env.close()
        cls = DummyVectorEnv if self.vector_env == "dummy" else SubprocVectorEnv
        self.env = cls(self._factories(task_ids))
        self._env_tasks = list(task_ids)

    # ---- observations ----------------------------------------------------------------------------------------------
    def _pack(self, i: int, raw: Optional[Dict[str, Any]]) -> Dict[str, Any]:
        if raw is None:                 # slot not stepped this call: its last observation stands
            out = dict(self._last[i])
        else:
            out = {"image": LU.camera_frame(raw, "agentview_image"),
                   "wrist_image": LU.camera_frame(raw, "robot0_eye_in_hand_image"),
                   "state": LU.proprio_state(raw),
                   "task_description": self.benchmark.get_task(self.task_ids[i]).language}
        out.update(step=int(self.steps[i]), done=bool(self.done[i]), success=bool(self.success[i]))
        return out

    # ---- interface ---------------------------------------------------------------------------------------------------
    async def reset(self, task_ids=None, trial_ids=None) -> List[Dict[str, Any]]:
        task_ids = [int(t) for t in (task_ids if task_ids is not None else range(self.num_envs))]
        trial_ids = [int(t) for t in (trial_ids if trial_ids is not None else [0] * len(task_ids))]
        n = len(task_ids)
        assert n <= self.num_envs and len(trial_ids) == n
        self._ensure_envs(task_ids)
        self.task_ids = task_ids
        self.env.reset()
        inits = []
        for tid, trial in zip(task_ids, trial_ids):
            states = self.benchmark.get_task_init_states(tid)
            inits.append(states[trial % len(states)])
        raw = self.env.call("set_init_state", inits)
        noop = LU.dummy_action(self.model_family)
        for _ in range(self.num_steps_wait):
            raw = self.env.step([noop] * n)[0]
        self.steps = np.zeros(n, dtype=np.int64)
        self.done = np.zeros(n, dtype=bool)
        self.success = np.zeros(n, dtype=bool)
        self._last = [{} for _ in range(n)]
        self._last = [self._pack(i, raw[i]) for i in range(n)]
        return [dict(o) for o in self._last]

    async def step(self, action) -> List[Dict[str, Any]]:
        a = np.asarray(action["actions"] if isinstance(action, dict) else action, dtype=np.float32)
        if a.ndim == 2:
            a = a[:, None, :]
        n = len(self.task_ids)
        assert a.shape[0] == n, f"{a.shape[0]} action rows for {n} environments"
        rewards = np.zeros(n, dtype=np.float32)
        fresh: List[Optional[Dict[str, Any]]] = [None] * n
        for c in range(a.shape[1]):
            live = [i for i in range(n) if not self.done[i]]
            if not live:
                break
            cmds = [LU.policy_action_to_env(a[i, c], self.model_family).tolist() for i in live]
            ret = self.env.step(cmds, ids=live)
            if len(ret) == 5:           # gymnasium-style: terminated, truncated
                obs, rew, term, trunc, _ = ret
                solved = np.logical_or(term, trunc)
            else:
                obs, rew, solved, _ = ret
            for k, i in enumerate(live):
                self.steps[i] += 1
                rewards[i] += float(rew[k])
                fresh[i] = obs[k]
                if bool(solved[k]):
                    self.success[i] = True
                if bool(solved[k]) or self.steps[i] >= self.max_steps:
                    self.done[i] = True
        out = []
        for i in range(n):
            o = self._pack(i, fresh[i])
            o["reward"] = float(rewards[i])
            self._last[i] = {k: v for k, v in o.items() if k != "reward"}
            out.append(o)
        return out

    def close(self) -> None:
        if self.env is not None:
            self.env.close()
            self.env = None
            self._env_tasks = None
