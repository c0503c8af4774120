from .base import BaseVLAEnvironment  # noqa: F401
from .synthetic import SyntheticReachEnv  # noqa: F401
from .venv import DummyVectorEnv, SubprocVectorEnv  # noqa: F401


def make_environment(env_type: str, **kwargs) -> BaseVLAEnvironment:
    """``synthetic`` (headless) or ``libero`` (needs robosuite + a GL renderer)."""
    if env_type == "synthetic":
        return SyntheticReachEnv(**{k: v for k, v in kwargs.items() if k in (
            "num_envs", "max_steps", "image_size", "device", "success_radius", "action_scale", "num_tasks")})
    if env_type == "libero":
        from .adapters.libero import LIBEROAdapter
        return LIBEROAdapter(**kwargs)
    raise ValueError(f"unknown environment type '{env_type}'")
