from .embodied_actor import flatten_trajectories, scatter_steps  # noqa: F401
