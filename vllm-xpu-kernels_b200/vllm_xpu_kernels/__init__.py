"""B200 (sm_100a) implementation of the fused-MoE operators of vllm-xpu-kernels.

Importing ``vllm_xpu_kernels._C``, ``._moe_C`` or ``._xpu_C`` registers the
operators under ``torch.ops._C`` / ``._moe_C`` / ``._xpu_C`` on the CUDA
dispatch key, the way the reference's extension modules register them on XPU.
"""
__version__ = "0.1.0"
