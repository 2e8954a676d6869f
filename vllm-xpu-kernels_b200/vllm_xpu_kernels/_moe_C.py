"""Registers the torch.ops._moe_C operators of the fused-MoE path (CUDA)."""
from ._loader import load as _load

_load()
