"""Registers the torch.ops._xpu_C operators of the fused-MoE path (CUDA)."""
from ._loader import load as _load

_load()
