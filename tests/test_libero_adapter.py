"""LIBERO adapter against a stand-in for the ``libero`` package (the real one needs MuJoCo with an off-screen
renderer): initial states by trial, settle steps, gripper conventions, chunked stepping that leaves finished slots
alone, observation contents; plus the conventions module itself."""
import asyncio
import math
import sys
import types

import numpy as np
import pytest

from siirl_b200.utils.embodied import libero_utils as LU


class _FakeSim:
    log = []                      # (task, action) of every simulator step, across instances

    def __init__(self, bddl_file_name, camera_heights, camera_widths, render_gpu_device_id):
        self.task = int(bddl_file_name.rsplit("task", 1)[1].split(".")[0])
        self.res = camera_heights
        self.x = 0.0

    def _obs(self):
        img = np.zeros((self.res, self.res, 3), dtype=np.uint8)
        img[0, 0] = 255                                   # a marker in the top-left corner of the raw render
        return {"agentview_image": img, "robot0_eye_in_hand_image": img // 2,
                "robot0_eef_pos": np.array([self.x, 0.0, 1.0]), "robot0_eef_quat": np.array([0.0, 0.0, 0.0, 1.0]),
                "robot0_gripper_qpos": np.array([0.02, -0.02])}

    def reset(self):
        self.x = 0.0
        return self._obs()

    def set_init_state(self, s):
        self.x = float(s)
        return self._obs()

    def step(self, a):
        _FakeSim.log.append((self.task, list(a)))
        self.x += float(a[0])
        return self._obs(), 1.0 if self.x >= 1.0 else 0.0, self.x >= 1.0, {}

    def close(self):
        pass


@pytest.fixture
def fake_libero(monkeypatch):
    class Task:
        def __init__(self, i):
            self.problem_folder, self.bddl_file, self.language = "suite", f"task{i}.bddl", f"do thing {i}"

    class Suite:
        def get_task(self, i):
            return Task(i)

        def get_task_init_states(self, i):
            return [0.0, 0.25, 0.5]

    root, inner, envs = types.ModuleType("libero"), types.ModuleType("libero.libero"), types.ModuleType("libero.libero.envs")
    inner.benchmark = types.SimpleNamespace(get_benchmark_dict=lambda: {"libero_goal": Suite})
    inner.get_libero_path = lambda key: "/nowhere"
    envs.OffScreenRenderEnv = _FakeSim
    root.libero, inner.envs = inner, envs
    for name, mod in (("libero", root), ("libero.libero", inner), ("libero.libero.envs", envs)):
        monkeypatch.setitem(sys.modules, name, mod)
    _FakeSim.log = []
    return Suite


def _run(coro):
    loop = asyncio.new_event_loop()
    try:
        return loop.run_until_complete(coro)
    finally:
        loop.close()


def test_adapter_reset_step_and_conventions(fake_libero):
    from siirl_b200.environment.embodied import make_environment
    env = make_environment("libero", env_name="libero_goal", num_envs=2, max_steps=6, num_steps_wait=3,
                           model_family="openvla", resolution=8, vector_env="dummy")
    obs = _run(env.reset([4, 7], [1, 5]))                 # trial 5 wraps around the three recorded states
    assert [o["task_description"] for o in obs] == ["do thing 4", "do thing 7"]
    assert len(_FakeSim.log) == 2 * 3 and all(a == LU.DUMMY_ACTION for _, a in _FakeSim.log)
    assert obs[0]["state"].shape == (8,) and abs(obs[0]["state"][0] - 0.25) < 1e-6 and abs(obs[1]["state"][0] - 0.5) < 1e-6
    assert obs[0]["image"][-1, -1, 0] == 255 and obs[0]["image"][0, 0, 0] == 0        # rotated by 180 degrees
    assert obs[0]["wrist_image"][-1, -1, 0] == 127 and not obs[0]["done"] and obs[0]["step"] == 0
    _FakeSim.log = []
    chunk = np.zeros((2, 4, 7), dtype=np.float32)
    chunk[0, :, 0] = 0.3                                   # slot 0 reaches x >= 1 at its third action: 0.25 + 0.9
    chunk[1, :, 0] = 0.01
    chunk[:, :, 6] = [[1.0, 0.6, 0.4, 0.0]] * 2            # policy gripper in [0, 1]: open .. close
    out = _run(env.step(chunk))
    assert out[0]["done"] and out[0]["success"] and out[0]["step"] == 3 and out[0]["reward"] == 1.0
    assert not out[1]["done"] and out[1]["step"] == 4
    steps0 = [a for t, a in _FakeSim.log if t == 4]
    assert len(steps0) == 3 and len([a for t, a in _FakeSim.log if t == 7]) == 4        # slot 0 not stepped when done
    assert [a[6] for t, a in _FakeSim.log if t == 7] == [-1.0, -1.0, 1.0, 1.0]          # 2g-1, sign, flipped
    out = _run(env.step(chunk[:, :2]))                     # the finished slot stays as it was; slot 1 hits max_steps
    assert out[0]["step"] == 3 and out[0]["done"] and out[1]["step"] == 6 and out[1]["done"] and not out[1]["success"]
    assert out[0]["image"] is not None and out[0]["reward"] == 0.0
    n_before = len(_FakeSim.log)
    _run(env.step(chunk[:, :1]))
    assert len(_FakeSim.log) == n_before                   # nothing is live: no simulator is stepped
    sims = env.env.envs
    _run(env.reset([4, 7], [0, 0]))
    assert env.env.envs is sims                            # same tasks: the simulators are kept
    env.close()
    with pytest.raises(ValueError):
        make_environment("libero", env_name="libero_nonexistent", vector_env="dummy")


def test_conventions_module(tmp_path):
    a = np.array([0.1, 0, 0, 0, 0, 0, 0.8], dtype=np.float32)
    assert LU.normalize_gripper_action(a)[-1] == 1.0 and LU.normalize_gripper_action(a, binarize=False)[-1] == pytest.approx(0.6)
    assert LU.invert_gripper_action(LU.normalize_gripper_action(a))[-1] == -1.0 and a[-1] == pytest.approx(0.8)
    assert LU.policy_action_to_env(a, "native")[-1] == 1.0
    assert np.allclose(LU.quat2axisangle([0, 0, 0, 1]), 0)
    half = math.sqrt(0.5)
    assert np.allclose(LU.quat2axisangle([half, 0, 0, half]), [math.pi / 2, 0, 0], atol=1e-6)
    frames = [np.full((8, 8, 3), i * 20, dtype=np.uint8) for i in range(4)]
    path = LU.save_rollout_video(frames, str(tmp_path), "Pick up: the block!", 12, True, fps=10)
    assert "step=12--success=True--task=pick_up__the_block_" in path
    import os
    assert os.path.getsize(path) > 0


def test_unavailable_without_the_package():
    from siirl_b200.environment.embodied.adapters.libero import EnvironmentUnavailable, LIBEROAdapter
    if "libero" in sys.modules:
        pytest.skip("a libero package is importable here")
    with pytest.raises(EnvironmentUnavailable):
        LIBEROAdapter()
