"""Fused Mixture-of-Experts layer for B200.

``XpuFusedMoe`` keeps the constructor and ``apply`` signature of
vllm_xpu_kernels/fused_moe_interface.py:186-330 of the reference project, so
vLLM code that drives that class runs unchanged; underneath, every step is a
hand-written sm_100a kernel:

    remap_hidden_states  ->  grouped GEMM w13 (+ gated activation in the
    epilogue where the recipe allows)  ->  [activation quant]  ->  grouped GEMM
    w2  ->  moe_gather

Recipes, detected from the weight dtypes as the reference does
(fused_moe_interface.py:70-83):

* bf16 / fp16 weights ``[E, K, N]``: tcgen05 kind::f16, activation fused into
  the first GEMM's epilogue.
* block-FP8 weights ``[E, K, N]`` + f32 scales ``[E, K/128, N/128]``:
  activations are FP8 with one f32 scale per token per 128 columns (passed in
  as ``a1q_scale`` or quantised here), tcgen05 kind::f8f6f4 with the scales
  applied per 128 of K; SiLU*mul and the re-quantisation for the second GEMM are
  one fused kernel.
* MXFP4 weights ``[E, N, K/2]`` + e8m0 scales ``[E, N, K/32]``: the weights stay
  4-bit in memory.  Activations are quantised to MXFP8 (e4m3 with one e8m0
  scale per 32 columns, the quantisation moe_utils.py:84-109 of the reference
  applies to activations) and both scale sets are applied inside tcgen05.mma
  kind::mxf8f6f4.block_scale; SwigluOAI and the re-quantisation for the second
  GEMM run in the first GEMM's epilogue.  ``VLLM_XPU_FUSED_MOE_USE_MXFP4_FP8``
  (the reference's ``mxfp4_fp8`` recipe: FP8 activations on MXFP4 weights)
  selects the same path.  ``B200MOE_MXFP4_W4A16=1`` gives the W4A16 arithmetic
  of the reference kernel instead: weights expanded once, exactly, to bf16
  ``[E, N, K]`` (every e2m1 x 2^e product is a bf16 number), bf16 activations.
"""
import contextlib
import math
import os
from typing import Optional

import torch

try:
    from . import _C  # noqa: F401
    from . import _moe_C  # noqa: F401
    from . import _xpu_C  # noqa: F401
    FUSEDMOE_UNAVAILABLE_REASON = None
    FUSEDMOE_AVAILABLE = True
except ImportError as e:  # the class below then raises on construction
    FUSEDMOE_UNAVAILABLE_REASON = str(e)
    FUSEDMOE_AVAILABLE = False

EPI_STORE, EPI_SILU_MUL, EPI_SWIGLU_OAI = 0, 1, 2
B_LAYOUT_KN, B_LAYOUT_NK = 0, 1
A_SCALE_ROW_MAJOR_DECODE = 2   # row-major activation scales + the decode-regime GEMM kernel


def _get_weights_dtype(weight, scales):
    dt = weight.dtype
    is_fp8 = dt in (torch.float8_e4m3fn, torch.float8_e5m2)
    is_int4 = dt == torch.uint8
    is_mxfp4 = dt == torch.float4_e2m1fn_x2
    is_mxfp8 = is_fp8 and scales is not None and scales.dtype in (torch.uint8, torch.float8_e8m0fnu)
    is_block_fp8 = (is_fp8 and scales is not None and scales.dtype == torch.float32
                    and scales.ndim == 3)
    is_fp8 = is_fp8 and not is_mxfp8 and not is_block_fp8
    return is_fp8, is_int4, is_mxfp4, is_mxfp8, is_block_fp8


USE_MXFP4_FP8_ENV = "VLLM_XPU_FUSED_MOE_USE_MXFP4_FP8"


def _is_env_enabled(name: str, default: str = "0") -> bool:
    return os.environ.get(name, default).strip().upper() in ("1", "ON", "TRUE", "YES", "Y")


def _get_recipe(is_fp8, is_mxfp8, is_mxfp4, is_int4, is_block_fp8):
    if is_mxfp8:
        return "mxfp8"
    if is_block_fp8:
        return "fp8block"
    if is_mxfp4:
        return "mxfp4_fp8" if _is_env_enabled(USE_MXFP4_FP8_ENV) else "mxfp4"
    if is_int4:
        return "int4"
    if is_fp8:
        return "fp8"
    return "bf16"


# activation name -> code of b200_act_and_mul (swigluoai has an op of its own)
_ACT_CODES = {"silu": 0, "gelu": 1, "gelu_tanh": 2, "swiglustep": 3, "situ": 4, "relu2_no_mul": 5,
              "swigluoai": -1}


def _is_swigluoai(activation) -> bool:
    return activation == "swigluoai" or "SWIGLUOAI" in str(activation)


class XpuFusedMoe:

    def __init__(
        self,
        w13,
        w13_scales,
        w13_bias,
        w2,
        w2_scales,
        w2_bias,
        n_experts_per_token,
        activation,
        num_experts,
        ep_rank=0,
        ep_size=1,
        expert_map=None,
        gemm1_clamp_limit: Optional[float] = None,
        activation_situ_beta: Optional[float] = None,
        activation_situ_linear_beta: Optional[float] = None,
    ):
        if not FUSEDMOE_AVAILABLE:
            raise ImportError(FUSEDMOE_UNAVAILABLE_REASON)
        assert w13.is_contiguous() and w2.is_contiguous()
        assert w13.is_cuda, "XpuFusedMoe (B200) needs its weights on a CUDA device"
        flags = _get_weights_dtype(w13, w13_scales)
        self.is_fp8, self.is_int4, self.is_mxfp4, self.is_mxfp8, self.is_block_fp8 = flags
        self.recipe = _get_recipe(self.is_fp8, self.is_mxfp8, self.is_mxfp4, self.is_int4,
                                  self.is_block_fp8)
        self._act_code = _ACT_CODES.get("swigluoai" if _is_swigluoai(activation) else activation)
        if self._act_code is None:
            raise ValueError(f"Unsupported FusedMoe activation: {activation}.")
        self.activation_situ_beta = activation_situ_beta
        self.activation_situ_linear_beta = activation_situ_linear_beta
        if activation == "situ":
            # same checks and texts as fused_moe_interface.py:253-262 of the reference
            if activation_situ_beta is None:
                raise ValueError("SITU requires activation_situ_beta")
            if not math.isfinite(activation_situ_beta):
                raise ValueError("SITU activation_situ_beta must be finite")
            if activation_situ_beta <= 0:
                raise ValueError("SITU activation_situ_beta must be positive")
        # relu2_no_mul is not gated: the second GEMM contracts over all 2*inter columns
        self.inter_size_scale = 2 if activation == "relu2_no_mul" else 1

        # 4-bit weights are [E, N, K/2]; everything else is [E, K, N].
        self.inter_size = (w13.shape[-2] if (self.is_mxfp4 or self.is_int4) else w13.shape[-1]) // 2
        self.w13, self.w2 = w13, w2
        self.gemm1_wei_scales = w13_scales if self.recipe != "bf16" else None
        self.gemm2_wei_scales = w2_scales if self.recipe != "bf16" else None
        # Block-FP8 weights whose 128x128 scales are all exact powers of two (UE8M0-scaled
        # checkpoints) take the kernel that lets the tensor core apply the scales; the layer then
        # also quantises its activations with power-of-two scales.  Checked once, here (one
        # host read).  B200MOE_FP8_PROMOTE=1 keeps the general kernel.
        self.act_scales_pow2 = False
        if self.is_block_fp8 and not os.environ.get("B200MOE_FP8_PROMOTE"):
            def _pow2(t):
                m, _ = torch.frexp(t.float())
                return bool(((m == 0.5) & (t > 0)).all().item())
            H_, I2_ = w13.shape[-2], w13.shape[-1]
            dims_ok = H_ % 128 == 0 and (I2_ // 2) % 128 == 0
            self.act_scales_pow2 = dims_ok and _pow2(w13_scales) and _pow2(w2_scales)
            if dims_ok and not self.act_scales_pow2 and _is_env_enabled("B200MOE_FP8_REQUANT_POW2"):
                # opt-in load-time step: arbitrary fp32 block scales rounded up to powers of two,
                # the weights re-rounded against them, IN PLACE (one more e4m3 rounding per weight)
                from .moe_utils import requant_fp8_block_weights_pow2_
                requant_fp8_block_weights_pow2_(w13, w13_scales)
                requant_fp8_block_weights_pow2_(w2, w2_scales)
                self.act_scales_pow2 = True
        # W8A16 / W4A16 recipes: widened once per activation dtype, on first use
        self._expanded = {}
        self.w13_bias, self.w2_bias = w13_bias, w2_bias
        self.n_experts_per_token = n_experts_per_token
        self.activation = activation
        self.num_experts = num_experts
        self.ep_rank, self.ep_size = ep_rank, ep_size
        self.gemm1_clamp_limit = gemm1_clamp_limit

        self._mx_native = False
        if self.is_mxfp4:
            hidden = w13.shape[-1] * 2
            # the block-scaled tensor-core path reads packed 4-bit rows with TMA: 32-byte row pitch
            self._mx_native = (hidden % 64 == 0 and self.inter_size % 64 == 0 and hidden >= 128
                               and self.inter_size >= 128 and activation != "relu2_no_mul"
                               and (self.recipe == "mxfp4_fp8"
                                    or not _is_env_enabled("B200MOE_MXFP4_W4A16")))
            if self._mx_native:
                # weight scales rearranged once into the order the tensor core reads them
                self._w13_sf = torch.ops._xpu_C.b200_mx_prepare_weight_scales(
                    w13_scales.view(torch.uint8), hidden)
                self._w2_sf = torch.ops._xpu_C.b200_mx_prepare_weight_scales(
                    w2_scales.view(torch.uint8), self.inter_size)
            else:
                # W4A16: one-time exact expansion to bf16
                self._w13_16 = torch.ops._xpu_C.b200_dequant_weights(
                    w13.view(torch.uint8), w13_scales.view(torch.uint8))
                self._w2_16 = torch.ops._xpu_C.b200_dequant_weights(
                    w2.view(torch.uint8), w2_scales.view(torch.uint8))

        # Optional list; when set, apply() appends (stage, start_event, end_event)
        # for each stage, the way the reference's benchmark brackets its stages
        # (benchmark/src/fused_moe_interface_.py:84-168 there).
        self.stage_timer = None
        self.stage_only = None   # optional set of stage names to restrict the timer to

        self.expert_map = expert_map
        if self.expert_map is None and self.ep_size > 1:
            self.expert_map = torch.empty((self.num_experts * self.ep_size), dtype=torch.int32,
                                          device=w13.device)
            torch.ops._moe_C.init_expert_map(self.expert_map, self.num_experts, self.ep_rank,
                                             self.ep_size)
        if self.expert_map is not None:
            self.total_experts_num = self.expert_map.shape[0]
        else:
            self.total_experts_num = self.num_experts * self.ep_size
        self.local_experts_num = self.num_experts

    @contextlib.contextmanager
    def _stage(self, name):
        if self.stage_timer is None or (self.stage_only is not None and name not in self.stage_only):
            yield
            return
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        yield
        end.record()
        self.stage_timer.append((name, start, end))

    def launches_per_apply(self, num_rows: int) -> int:
        """Kernels one apply() enqueues for `num_rows` already-quantised tokens."""
        permute = 2 if num_rows * self.n_experts_per_token <= 2048 else 4
        return permute + 3  # gemm1 (activation [+ quantisation] fused), gemm2, gather

    # ------------------------------------------------------------------
    def apply(self, output, hidden_states, topk_weights, topk_ids, expert_map=None,
              a1q_scale=None, row_destinations=None, shared_output=None, valid_tokens=None,
              after_gemms=None):
        """output[T, H] = sum_j w[t, j] * Expert_{ids[t, j]}(hidden_states[t]).

        ``hidden_states`` is bf16/fp16 ``[T, H]``, or already quantised
        (e4m3 ``[T, H]`` with ``a1q_scale`` f32 ``[T, H/128]``) for block-FP8
        weights.  ``topk_weights`` is f32 ``[T, k]``; ``topk_ids`` int32/int64
        global expert ids; ``expert_map`` int32 global -> local id or -1.

        ``row_destinations`` (not in the reference signature; used by the expert-parallel
        exchange): a callable that gets the ``[T, k]`` row map and returns an int64 device
        table with, per permuted row, the address the second GEMM must store that row at.
        ``output`` is then not written and the weighted combine is the caller's.

        ``shared_output`` (not in the reference signature): ``[T, H]`` rows added to the
        routed result inside the combine, weight 1 - the output of a shared expert every
        token passes through (see ``dense``).

        ``valid_tokens`` (not in the reference signature; used by the expert-parallel token
        exchange): int32 ``[1]`` on the device, the number of leading rows of a worst-case
        sized ``hidden_states`` that hold tokens.  Rows past it must carry ids of -1; their
        output rows are then not written at all.

        ``after_gemms`` (not in the reference signature): a ``torch.cuda.Event`` recorded on the
        current stream right after the second grouped GEMM, before the combine."""
        num_rows, hidden_size = hidden_states.shape
        k = topk_ids.shape[1]  # n_experts_per_token, or 1 for rows that arrive already dispatched
        R = num_rows * k
        dev = hidden_states.device
        if expert_map is None and self.ep_size > 1:
            expert_map = self.expert_map
        if num_rows == 0:
            return

        if (self.is_block_fp8 and row_destinations is None and valid_tokens is None
                and self._decode_regime(num_rows * k)
                and self.activation == "silu" and not (self.gemm1_clamp_limit or 0) > 0
                and self.inter_size % 128 == 0):
            return self._apply_decode(output, hidden_states, topk_weights, topk_ids, expert_map,
                                      a1q_scale, shared_output)
        if self.is_block_fp8 and a1q_scale is None:
            # dynamic per-token-group-128 quantisation, once per token (not per routed row)
            from .moe_utils import quant_fp8_block_act
            hidden_states, a1q_scale = quant_fp8_block_act(hidden_states, self.act_scales_pow2)
        if self._mx_native:
            if a1q_scale is None:
                hidden_states, a1q_scale = torch.ops._xpu_C.b200_quant_mxfp8(hidden_states)
            else:
                a1q_scale = self._pad_mx_scales(a1q_scale, hidden_size)
        act_quant = a1q_scale is not None
        if act_quant and not (self.is_block_fp8 or self._mx_native):
            raise NotImplementedError(
                "quantised activations are taken with block-FP8 weights and on the MXFP4 tensor-core path")

        remapped = torch.empty((R, hidden_size), dtype=hidden_states.dtype, device=dev)
        remapped_scales = (torch.empty((R, a1q_scale.shape[1]), dtype=a1q_scale.dtype, device=dev)
                           if act_quant else None)
        rows_per_expert = torch.zeros((self.num_experts,), dtype=torch.int32, device=dev)
        row_map = torch.empty((num_rows, k), dtype=torch.int32, device=dev)
        with self._stage("remap"):
            torch.ops._moe_C.remap_hidden_states(hidden_states, a1q_scale, remapped,
                                                 remapped_scales, expert_map, rows_per_expert,
                                                 row_map, topk_ids, self.total_experts_num,
                                                 self.local_experts_num)

        row_ptr = row_destinations(row_map) if row_destinations is not None else None
        gemm2_out = self.run_experts(remapped, remapped_scales, rows_per_expert, output.dtype, row_ptr)
        if after_gemms is not None:
            after_gemms.record()
        if row_ptr is not None:
            return
        with self._stage("gather"):
            if shared_output is not None:
                torch.ops._moe_C.b200_moe_gather_add(output, gemm2_out, topk_weights, row_map,
                                                     shared_output)
            elif valid_tokens is not None:
                torch.ops._moe_C.b200_moe_gather_bounded(output, gemm2_out, topk_weights, row_map,
                                                         valid_tokens)
            else:
                torch.ops._moe_C.moe_gather(output, gemm2_out, topk_weights, row_map,
                                            self.num_experts)

    def dense(self, hidden_states, a1q_scale=None, out_dtype=torch.bfloat16):
        """A layer built with one expert used as a plain gated MLP over all rows: the shared
        expert of a DeepSeek-V3-style layer (the reference project has no operator for it; it
        is the grouped GEMM with a single group).  Returns ``[T, H]``; pass it to ``apply`` of
        the routed layer as ``shared_output``."""
        assert self.num_experts == 1, "dense() is for a layer built with a single expert"
        T = hidden_states.shape[0]
        if self.is_block_fp8 and a1q_scale is None:
            from .moe_utils import quant_fp8_block_act
            hidden_states, a1q_scale = quant_fp8_block_act(hidden_states, self.act_scales_pow2)
        elif self._mx_native and a1q_scale is None:
            hidden_states, a1q_scale = torch.ops._xpu_C.b200_quant_mxfp8(hidden_states)
        rows = getattr(self, "_dense_rows", None)
        if rows is None or rows[0] != T:
            rows = (T, torch.full((1,), T, dtype=torch.int32, device=hidden_states.device))
            self._dense_rows = rows
        return self.run_experts(hidden_states, a1q_scale, rows[1], out_dtype)

    def run_experts(self, rows, row_scales, rows_per_expert, out_dtype, row_ptr=None, out=None):
        """The two grouped GEMMs with the activation between them on rows that are already
        grouped by local expert (``rows_per_expert`` int32 on the device, experts back to
        back).  Returns the ``[R, H]`` result in the same row order, or, with ``row_ptr``
        (int64 address per row), stores each result row at its address and returns a
        placeholder.  ``out`` (``[R, H]``) is used as the result buffer when given.  Not part
        of the reference class; ``apply`` and the expert-parallel exchange both end here."""
        R, hidden_size = rows.shape
        dev = rows.device
        remapped, remapped_scales = rows, row_scales
        I, E = self.inter_size, self.num_experts
        oai = _is_swigluoai(self.activation)
        gemm = torch.ops._xpu_C.b200_grouped_gemm
        clamp = self.gemm1_clamp_limit is not None and self.gemm1_clamp_limit > 0
        if self._mx_native:
            if row_ptr is not None:
                raise NotImplementedError("per-row destinations are not taken on the MXFP4 tensor-core path")
            return self._run_experts_mx(rows, row_scales, rows_per_expert, out_dtype, out, oai, clamp)
        if self.is_block_fp8:
            K2 = I * self.inter_size_scale
            pow2 = self.act_scales_pow2
            fused = self._fused_gated(clamp)
            if (fused is not None and I % 128 == 0 and not os.environ.get("B200MOE_UNFUSED_ACT")):
                # activation * up (with the layer's clamp) and the group-128 re-quantisation run
                # in the GEMM's epilogue
                act_q = torch.empty((R, I), dtype=torch.float8_e4m3fn, device=dev)
                act_s = torch.empty((R, I // 128), dtype=torch.float32, device=dev)
                with self._stage("gemm1"):
                    gemm(remapped, remapped_scales, self.w13, self.gemm1_wei_scales, self.w13_bias,
                         act_q, rows_per_expert, 2 * I, hidden_size, E, EPI_SILU_MUL, B_LAYOUT_KN,
                         1.702, 7.0, act_s, None, 0, *fused, pow2)
            else:
                gemm1_out = torch.empty((R, 2 * I), dtype=out_dtype, device=dev)
                with self._stage("gemm1"):
                    gemm(remapped, remapped_scales, self.w13, self.gemm1_wei_scales, self.w13_bias,
                         gemm1_out, rows_per_expert, 2 * I, hidden_size, E, EPI_STORE, B_LAYOUT_KN,
                         1.702, 7.0, None, None, 0, 0, 0.0, 0.0, 0.0, pow2)
                act_q = torch.empty((R, K2), dtype=torch.float8_e4m3fn, device=dev)
                act_s = torch.empty((R, K2 // 128), dtype=torch.float32, device=dev)
                with self._stage("act_quant"):
                    if self.activation == "silu" and not clamp and not pow2:
                        torch.ops._C.silu_and_mul_per_block_quant(act_q, gemm1_out, act_s, 128)
                    else:
                        act = self._activate(gemm1_out)
                        torch.ops._C.per_token_group_fp8_quant(act, act_q, act_s, 128, 1e-10, -448.0,
                                                               448.0, pow2, False, False)
            gemm2_out = out if out is not None else torch.empty(
                (R if row_ptr is None else 1, hidden_size), dtype=out_dtype, device=dev)
            with self._stage("gemm2"):
                gemm(act_q, act_s, self.w2, self.gemm2_wei_scales, self.w2_bias, gemm2_out,
                     rows_per_expert, hidden_size, K2, E, EPI_STORE, B_LAYOUT_KN, 1.702, 7.0, None,
                     row_ptr, 0, 0, 0.0, 0.0, 0.0, pow2 and K2 % 128 == 0)
        else:
            w13, w2, layout = self._weights_16(out_dtype)
            K2 = I * self.inter_size_scale
            fused = self._fused_gated(clamp)
            fused_epi = (fused is not None or oai) and not os.environ.get("B200MOE_UNFUSED_ACT")
            if fused_epi:
                lim = float(self.gemm1_clamp_limit) if clamp else 0.0
                extra = fused if fused is not None else (0, 0.0, 0.0, lim)
                act = torch.empty((R, I), dtype=out_dtype, device=dev)
                with self._stage("gemm1"):
                    gemm(remapped, None, w13, None, self.w13_bias, act, rows_per_expert, 2 * I,
                         hidden_size, E, EPI_SWIGLU_OAI if oai else EPI_SILU_MUL, layout, 1.702,
                         7.0, None, None, 0, *extra)
            else:
                gemm1_out = torch.empty((R, 2 * I), dtype=out_dtype, device=dev)
                with self._stage("gemm1"):
                    gemm(remapped, None, w13, None, self.w13_bias, gemm1_out, rows_per_expert,
                         2 * I, hidden_size, E, EPI_STORE, layout)
                with self._stage("act"):
                    act = self._activate(gemm1_out)
            gemm2_out = out if out is not None else torch.empty(
                (R if row_ptr is None else 1, hidden_size), dtype=out_dtype, device=dev)
            with self._stage("gemm2"):
                gemm(act, None, w2, None, self.w2_bias, gemm2_out, rows_per_expert, hidden_size, K2,
                     E, EPI_STORE, layout, 1.702, 7.0, None, row_ptr)
        return gemm2_out

    def _fused_gated(self, clamp):
        """(activation code, param0, param1, clamp limit) when the activation is one the first
        GEMM's split gated epilogue evaluates (act(gate) * up on the fp32 accumulators, with
        the layer's clamp before it), else None (swigluoai has an epilogue of its own;
        relu2_no_mul is not gated)."""
        if self._act_code < 0 or self.activation == "relu2_no_mul" or self.inter_size_scale != 1:
            return None
        p0 = p1 = 0.0
        if self.activation == "swiglustep":
            p0 = 7.0
        elif self.activation == "situ":
            p0 = self.activation_situ_beta
            p1 = -1.0 if self.activation_situ_linear_beta is None else self.activation_situ_linear_beta
        lim = float(self.gemm1_clamp_limit) if clamp else 0.0
        return (self._act_code, float(p0), float(p1), lim)

    @staticmethod
    def _pad_mx_scales(scales, width):
        """e8m0 scales [T, width/32] (uint8 or float8_e8m0fnu) -> uint8 [T, 16*ceil(width/512)],
        the row pitch the block-scaled GEMM reads 16 bytes at a time."""
        sf = scales.view(torch.uint8)
        pitch = (width + 511) // 512 * 16
        if sf.shape[1] == pitch:
            return sf.contiguous()
        out = torch.full((sf.shape[0], pitch), 127, dtype=torch.uint8, device=sf.device)
        out[:, :width // 32] = sf[:, :width // 32]
        return out

    def _run_experts_mx(self, rows, row_sf, rows_per_expert, out_dtype, out, oai, clamp):
        """MXFP8 rows x MXFP4 weights on the block-scaled tensor-core path."""
        R, H = rows.shape
        dev = rows.device
        I, E = self.inter_size, self.num_experts
        gemm = torch.ops._xpu_C.b200_grouped_gemm_mx
        w13, w2 = self.w13.view(torch.uint8), self.w2.view(torch.uint8)
        pitch_i = (I + 511) // 512 * 16
        if oai and not clamp:
            # SwigluOAI and the MXFP8 quantisation of its result run in the GEMM's epilogue
            act_q = torch.empty((R, I), dtype=torch.float8_e4m3fn, device=dev)
            act_sf = torch.empty((R, pitch_i), dtype=torch.uint8, device=dev)
            with self._stage("gemm1"):
                gemm(rows, row_sf, w13, self._w13_sf, self.w13_bias, act_q, act_sf, rows_per_expert,
                     2 * I, H, E, EPI_SWIGLU_OAI, 1.702, 7.0)
        else:
            gemm1_out = torch.empty((R, 2 * I), dtype=out_dtype, device=dev)
            with self._stage("gemm1"):
                gemm(rows, row_sf, w13, self._w13_sf, self.w13_bias, gemm1_out, None, rows_per_expert,
                     2 * I, H, E, EPI_STORE, 1.702, 7.0)
            with self._stage("act_quant"):
                act_q, act_sf = torch.ops._xpu_C.b200_quant_mxfp8(self._activate(gemm1_out))
        gemm2_out = out if out is not None else torch.empty((R, H), dtype=out_dtype, device=dev)
        with self._stage("gemm2"):
            gemm(act_q, act_sf, w2, self._w2_sf, self.w2_bias, gemm2_out, None, rows_per_expert, H, I, E,
                 EPI_STORE, 1.702, 7.0)
        return gemm2_out

    def _decode_regime(self, routed_rows: int) -> bool:
        """Whether to run the two GEMMs on the decode-regime kernel (weights on the M side of
        the MMA, 32 tokens per tile).  With at most about one routed row per local expert it is
        4-6 % faster end to end on the DeepSeek-V3 shape (1..32 tokens); from a few rows per
        expert on, hot experts need several 32-token chunks that each stream the weights again,
        and the 128-row-tile kernel wins.  B200MOE_DECODE_PATH=0/1 overrides."""
        forced = os.environ.get("B200MOE_DECODE_PATH")
        if forced is not None:
            return forced == "1"
        return routed_rows <= self.num_experts

    def _apply_decode(self, output, hidden_states, topk_weights, topk_ids, expert_map, a1q_scale,
                      shared_output=None):
        """Same sequence of launches as the default path, with the two grouped GEMMs on the
        decode-regime kernel (weights on the M side of the MMA, 32 tokens per tile); the first
        one quantises its output per token per 128 columns in its epilogue."""
        from .moe_utils import quant_fp8_block_act
        T, H = hidden_states.shape
        k = topk_ids.shape[1]
        R, I, E = T * k, self.inter_size, self.num_experts
        dev = hidden_states.device
        if a1q_scale is None:
            hidden_states, a1q_scale = quant_fp8_block_act(hidden_states)
        if expert_map is None and self.ep_size > 1:
            expert_map = self.expert_map
        remapped = torch.empty((R, H), dtype=hidden_states.dtype, device=dev)
        remapped_scales = torch.empty((R, a1q_scale.shape[1]), dtype=a1q_scale.dtype, device=dev)
        rows_per_expert = torch.zeros((E,), dtype=torch.int32, device=dev)
        row_map = torch.empty((T, k), dtype=torch.int32, device=dev)
        with self._stage("remap"):
            torch.ops._moe_C.remap_hidden_states(hidden_states, a1q_scale, remapped, remapped_scales,
                                                 expert_map, rows_per_expert, row_map, topk_ids,
                                                 self.total_experts_num, self.local_experts_num)
        gemm = torch.ops._xpu_C.b200_grouped_gemm
        act_q = torch.empty((R, I), dtype=torch.float8_e4m3fn, device=dev)
        act_s = torch.empty((R, I // 128), dtype=torch.float32, device=dev)
        with self._stage("gemm1"):
            gemm(remapped, remapped_scales, self.w13, self.gemm1_wei_scales, self.w13_bias, act_q,
                 rows_per_expert, 2 * I, H, E, EPI_SILU_MUL, B_LAYOUT_KN, 1.702, 7.0, act_s, None,
                 A_SCALE_ROW_MAJOR_DECODE)
        gemm2_out = torch.empty((R, H), dtype=output.dtype, device=dev)
        with self._stage("gemm2"):
            gemm(act_q, act_s, self.w2, self.gemm2_wei_scales, self.w2_bias, gemm2_out, rows_per_expert,
                 H, I, E, EPI_STORE, B_LAYOUT_KN, 1.702, 7.0, None, None, A_SCALE_ROW_MAJOR_DECODE)
        with self._stage("gather"):
            if shared_output is not None:
                torch.ops._moe_C.b200_moe_gather_add(output, gemm2_out, topk_weights, row_map,
                                                     shared_output)
            else:
                torch.ops._moe_C.moe_gather(output, gemm2_out, topk_weights, row_map, self.num_experts)

    def _weights_16(self, dtype):
        """(w13, w2, layout) as 16-bit operands of the grouped GEMM."""
        if self.recipe == "bf16":
            return self.w13, self.w2, B_LAYOUT_KN
        if self.is_mxfp4:
            return self._w13_16, self._w2_16, B_LAYOUT_NK
        if dtype not in self._expanded:
            expand = torch.ops._xpu_C.b200_expand_weights
            s13, s2 = self.gemm1_wei_scales, self.gemm2_wei_scales
            if self.recipe == "fp8":
                s13, s2 = (t.to(torch.float32).reshape(-1).contiguous() for t in (s13, s2))
            elif self.recipe == "mxfp8":
                s13, s2 = (t.view(torch.uint8) for t in (s13, s2))
            self._expanded[dtype] = (expand(self.w13, s13, self.recipe, dtype),
                                     expand(self.w2, s2, self.recipe, dtype))
        w13, w2 = self._expanded[dtype]
        return w13, w2, (B_LAYOUT_NK if self.is_int4 else B_LAYOUT_KN)

    def _activate(self, gemm1_out):
        """Activation as a pass of its own over the first GEMM's output, with the layer's
        clamp (gate <= limit, |up| <= limit; fused_moe_interface.py:436-441 of the reference)
        folded into the same kernel."""
        R = gemm1_out.shape[0]
        lim = self.gemm1_clamp_limit if (self.gemm1_clamp_limit or 0) > 0 else 0.0
        act = torch.empty((R, self.inter_size * self.inter_size_scale), dtype=gemm1_out.dtype,
                          device=gemm1_out.device)
        if self._act_code < 0:  # swigluoai: interleaved gate/up, limit of its own
            if lim:
                gemm1_out[:, :self.inter_size].clamp_(max=lim)
                gemm1_out[:, self.inter_size:].clamp_(min=-lim, max=lim)
            torch.ops._C.swigluoai_and_mul(act, gemm1_out, 1.702, 7.0)
            return act
        p0 = p1 = 0.0
        if self.activation == "swiglustep":
            p0 = 7.0
        elif self.activation == "situ":
            p0 = self.activation_situ_beta
            p1 = -1.0 if self.activation_situ_linear_beta is None else self.activation_situ_linear_beta
        torch.ops._C.b200_act_and_mul(act, gemm1_out, self._act_code, p0, p1, lim)
        return act
