"""The C-ABI library loads on a machine without a GPU and exports every symbol
that include/b200moe.h declares; the ctypes table covers the same set."""
import ctypes
import os
import re

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200moe.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200moe_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from vllm_xpu_kernels._loader import CAPI_PATH
    lib = ctypes.CDLL(CAPI_PATH)
    names = declared_symbols()
    assert len(names) >= 24
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/b200moe.h but not exported"


def test_ctypes_table_matches_header():
    from vllm_xpu_kernels import capi
    assert sorted(capi.SIGNATURES) == declared_symbols()
    assert capi.lib().b200moe_version().startswith(b"b200moe")
    assert capi.status_string(capi.TIMEOUT) == "device-side wait timed out"


def test_argument_checks_need_no_gpu():
    """Invalid-argument paths return before any CUDA call."""
    from vllm_xpu_kernels import capi
    lib = capi.lib()
    assert lib.b200moe_topk_softmax(None, capi.F32, 4, 8, 9, 1, None, None, None, None, capi.I32, None, None) == capi.INVALID_ARG
    assert lib.b200moe_grouped_topk(None, capi.F32, None, capi.F32, 4, 256, 7, 4, 8, 1, 2.5, 1, None, None, None) == capi.INVALID_ARG
    assert lib.b200moe_per_token_group_quant_mxfp4(None, capi.BF16, None, None, 4, 64, 16, 1e-10, 2, 1, None) == capi.UNSUPPORTED
    assert lib.b200moe_moe_align_block_size_workspace_bytes(100, 8) == 0
    assert lib.b200moe_moe_align_block_size_workspace_bytes(131072, 256) == 64 * 256 * 4
    a = capi.GemmArgs(recipe=capi.RECIPE_MXFP4, E=4, N=128, K=64)
    assert lib.b200moe_grouped_gemm_workspace_bytes(ctypes.byref(a)) == 4 * 128 * 64 * 2


def test_operator_schemas_are_registered():
    import torch
    import vllm_xpu_kernels._C  # noqa: F401
    import vllm_xpu_kernels._moe_C  # noqa: F401
    import vllm_xpu_kernels._xpu_C  # noqa: F401
    for ns, names in {"_moe_C": ["moe_sum", "moe_align_block_size", "grouped_topk", "topk_softmax",
                                 "topk_sigmoid", "moe_gather", "init_expert_map", "remap_hidden_states"],
                      "_C": ["silu_and_mul", "swigluoai_and_mul", "per_token_group_fp8_quant",
                             "per_token_group_quant_mxfp4", "silu_and_mul_per_block_quant",
                             "silu_and_mul_mxfp4_quant"],
                      "_xpu_C": ["cutlass_grouped_gemm_interface"]}.items():
        for n in names:
            assert hasattr(getattr(torch.ops, ns), n)
    # no CPU kernel exists: a CPU tensor must be refused, not silently computed
    import pytest
    with pytest.raises((RuntimeError, NotImplementedError)):
        torch.ops._C.silu_and_mul(torch.empty(2, 4), torch.zeros(2, 8))
