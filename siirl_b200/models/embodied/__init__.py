from .vla import ActionTokenizer, VLAProcessor  # noqa: F401
