"""Loads the native libraries that sit next to this file.

There is no Python or CPU implementation behind the operators: if the shared
objects are missing the import fails, and if a tensor is not on a CUDA device
the dispatcher has nothing to run.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
CAPI_PATH = os.path.join(_HERE, "libb200moe.so")
TORCH_OPS_PATH = os.path.join(_HERE, "_b200_torch_ops.so")
_loaded = False


def load():
    global _loaded
    if _loaded:
        return
    for path in (CAPI_PATH, TORCH_OPS_PATH):
        if not os.path.exists(path):
            raise ImportError(
                f"{path} is missing: build it with `python vllm-xpu-kernels_b200/build.py` "
                "(needs nvcc with sm_100a support)")
    ctypes.CDLL(CAPI_PATH, mode=ctypes.RTLD_GLOBAL)
    torch.ops.load_library(TORCH_OPS_PATH)
    _loaded = True
