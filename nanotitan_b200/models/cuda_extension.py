"""Accessor of the compiled extension under the reference's name (src/model/cuda_extension.py)."""
from nanotitan_b200.ops.ext import get_ext as get_cuda_extension

__all__ = ["get_cuda_extension"]
