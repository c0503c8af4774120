"""Operator layer: each op has a hand-written sm_100a CUDA kernel (used for every CUDA tensor)
and a plain-PyTorch statement (``reference``) used on CPU and as the test oracle."""
from . import reference  # noqa: F401
from .dense import (  # noqa: F401
    add, embedding, gemm, linear, rmsnorm, rope, rope_tables, swiglu,
)
