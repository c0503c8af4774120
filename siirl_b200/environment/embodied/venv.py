"""Vector environments for gym-style single environments: in-process (``DummyVectorEnv``) and one worker process
per environment (``SubprocVectorEnv``), the two modes of the reference's Tianshou-style implementation
(siirl/environment/embodied/venv.py:49-1028).  Observations come back as lists; numeric arrays are stacked."""
from __future__ import annotations

import multiprocessing as mp
from typing import Any, Callable, List, Optional, Sequence

import numpy as np


class DummyVectorEnv:
    def __init__(self, env_fns: Sequence[Callable[[], Any]]):
        self.envs = [fn() for fn in env_fns]
        self.env_num = len(self.envs)

    def __len__(self) -> int:
        return self.env_num

    def reset(self, ids: Optional[List[int]] = None, **kwargs):
        ids = list(range(self.env_num)) if ids is None else ids
        return [self.envs[i].reset(**kwargs) for i in ids]

    def step(self, actions, ids: Optional[List[int]] = None):
        ids = list(range(self.env_num)) if ids is None else ids
        outs = [self.envs[i].step(actions[k]) for k, i in enumerate(ids)]
        return tuple(_stack(x) for x in zip(*outs))

    def seed(self, seed: Optional[int] = None):
        return [e.seed(seed + i) if hasattr(e, "seed") and seed is not None else None for i, e in enumerate(self.envs)]

    def call(self, method: str, args: Sequence[Any], ids: Optional[List[int]] = None):
        """``env.method(args[k])`` on every listed environment (e.g. ``set_init_state``); returns the results."""
        ids = list(range(self.env_num)) if ids is None else ids
        return [getattr(self.envs[i], method)(args[k]) for k, i in enumerate(ids)]

    def close(self):
        for e in self.envs:
            if hasattr(e, "close"):
                e.close()


def _stack(xs):
    xs = list(xs)
    if isinstance(xs[0], (int, float, bool, np.number, np.ndarray)):
        return np.stack([np.asarray(x) for x in xs])
    return xs


def _worker(conn, fn):
    env = fn()
    try:
        while True:
            cmd, data = conn.recv()
            if cmd == "reset":
                conn.send(env.reset(**(data or {})))
            elif cmd == "step":
                conn.send(env.step(data))
            elif cmd == "seed":
                conn.send(env.seed(data) if hasattr(env, "seed") else None)
            elif cmd == "call":
                conn.send(getattr(env, data[0])(data[1]))
            elif cmd == "close":
                if hasattr(env, "close"):
                    env.close()
                conn.send(None)
                break
    except (EOFError, KeyboardInterrupt):
        pass


class SubprocVectorEnv:
    """One process per environment; ``step`` overlaps the environments' simulation."""

    def __init__(self, env_fns: Sequence[Callable[[], Any]], context: str = "spawn"):
        ctx = mp.get_context(context)
        self.env_num = len(env_fns)
        self.parents, self.procs = [], []
        for fn in env_fns:
            parent, child = ctx.Pipe()
            p = ctx.Process(target=_worker, args=(child, fn), daemon=True)
            p.start()
            child.close()
            self.parents.append(parent)
            self.procs.append(p)

    def __len__(self) -> int:
        return self.env_num

    def reset(self, ids: Optional[List[int]] = None, **kwargs):
        ids = list(range(self.env_num)) if ids is None else ids
        for i in ids:
            self.parents[i].send(("reset", kwargs))
        return [self.parents[i].recv() for i in ids]

    def step(self, actions, ids: Optional[List[int]] = None):
        ids = list(range(self.env_num)) if ids is None else ids
        for k, i in enumerate(ids):
            self.parents[i].send(("step", actions[k]))
        outs = [self.parents[i].recv() for i in ids]
        return tuple(_stack(x) for x in zip(*outs))

    def call(self, method: str, args: Sequence[Any], ids: Optional[List[int]] = None):
        ids = list(range(self.env_num)) if ids is None else ids
        for k, i in enumerate(ids):
            self.parents[i].send(("call", (method, args[k])))
        return [self.parents[i].recv() for i in ids]

    def close(self):
        for c in self.parents:
            try:
                c.send(("close", None))
                c.recv()
            except (BrokenPipeError, EOFError):
                pass
        for p in self.procs:
            p.join(timeout=5)
            if p.is_alive():
                p.terminate()
