"""ishizuki_b200: the speculative-decoding verify matmul of struffl/ishizuki for NVIDIA B200.

The product is libishizuki_cuda.so (CUDA for sm_100a behind the C ABI in
include/ishizuki_cuda.h). This package builds and loads it and mirrors, on top of it, the
reference's projection interface (PackedLinear, VerifyMatmul, GGMLKernels) for hosts and tests
written in Python.
"""
from . import build as build_module  # noqa: F401
from ._lib import load  # noqa: F401

__all__ = ["load", "build_module"]
