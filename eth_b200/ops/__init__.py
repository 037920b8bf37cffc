"""Ops of the GPT stage program: hand-written sm_100a kernels on CUDA, PyTorch references on CPU."""
from . import native  # noqa: F401
from .functional import *  # noqa: F401,F403
from .functional import gemm, colsum  # noqa: F401
