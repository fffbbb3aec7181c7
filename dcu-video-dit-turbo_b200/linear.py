"""INT8 linear orchestration behind the gates.

Mirror of `_int8_linear_nocopy` in the reference
(launcher/benchmark_launcher_v14_hires_int8_candidate.py:960-1067): apply the
input activation, quantise the activation rowwise, multiply by the int8 weight,
dequantise with row x column scales (+ bias), reshape.  Same argument meaning and
the same ValueErrors.  Two B200-specific routes are added in front of the
reference's three-kernel route, each behind its own gate:
  * swiglu input activation -> the fused swiglu-quant kernel (the hook the
    reference points at, :976);
  * GEMM + epilogue -> the single tcgen05 kernel with the epilogue fused, which
    skips the int32 [M,N] round trip.
ConvRot (launcher :993-999) has no kernel here: its Hadamard helpers belong to the host's
quantization package, which is not part of the reference tree, so the rotation cannot be
pinned.  `convrot=True` is therefore a counted refusal (reason `convrot`): the rotation of
the activation goes to the host's own helper, registered as the `convrot_rotate` fallback
`(x, groupsize) -> x`, and the rotated activation continues through the gated path below.
Without a registered helper the call raises, like every refusal without a fallback.
"""
from __future__ import annotations

import torch

from . import ops
from .gates import Gates, default_gates


def int8_linear(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                bias: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16,
                convrot: bool = False, convrot_groupsize: int = 256,
                input_act: str | None = None, gates: Gates | None = None) -> torch.Tensor:
    g = gates if gates is not None else default_gates()
    if convrot and input_act is not None:
        # the reference applies the input activation first and rotates its result
        x = g._fallback("input_act")(x, input_act)
        input_act = None
    k_in = x.shape[-1] // 2 if input_act == "swiglu" else x.shape[-1]
    if k_in != weight.shape[-1]:
        raise ValueError(
            f"Input and weight inner dimensions must match, got {k_in} and {weight.shape[-1]}")
    weight = weight.to(device=x.device)
    if not weight.is_contiguous():
        weight = weight.contiguous()
    weight_scale = weight_scale.to(device=x.device, dtype=torch.float32).reshape(-1)
    if weight_scale.numel() not in (1, weight.shape[0]):
        raise ValueError(
            f"INT8 weight scale must be scalar or per-output-channel, got "
            f"{tuple(weight_scale.shape)} for weight shape {tuple(weight.shape)}")

    if convrot:
        if x.shape[-1] % convrot_groupsize != 0:
            raise ValueError(
                f"ConvRot group size {convrot_groupsize} does not divide input features {x.shape[-1]}")
        g.counters["convrot"].refuse("convrot", x.shape, groupsize=convrot_groupsize)
        x = g._fallback("convrot_rotate")(x, convrot_groupsize)

    orig_shape = x.shape
    x_2d = x.reshape(-1, x.shape[-1])
    if input_act == "swiglu":
        x_8, x_scale = g.swiglu_quantize_activation(x_2d)
    elif input_act is None:
        x_8, x_scale = g.quantize_activation(x_2d, stochastic_rounding=0)
    else:
        x_8, x_scale = g.quantize_activation(g._fallback("input_act")(x_2d, input_act))

    col_scale = weight_scale
    if col_scale.numel() == 1:
        col_scale = col_scale.expand(weight.shape[0]).contiguous()
    else:
        col_scale = col_scale.contiguous()
    row_scale = x_scale.reshape(-1).contiguous()
    fused_bias = None if bias is None else bias.to(device=x.device).reshape(-1).contiguous()
    if fused_bias is not None and fused_bias.dtype not in (torch.bfloat16, torch.float32):
        fused_bias = fused_bias.to(torch.bfloat16)

    ok, reason = g.fused_gemm_gate(x_8, row_scale, weight, col_scale, fused_bias, out_dtype)
    if ok:
        g.counters["fused_gemm"].hit()
        result = ops.int8_gemm_dequant(x_8, row_scale, weight, col_scale, fused_bias)
        return result.reshape(*orig_shape[:-1], weight.shape[0])
    if g.fused_gemm_enabled:
        g.counters["fused_gemm"].refuse(reason, (x_8.shape[0], x_8.shape[1], weight.shape[0]))

    result = g.int8_matmul(x_8, weight.T)
    if g.epilogue_enabled and out_dtype == torch.bfloat16:
        vec4_ok, vec4_reason = g.vec4_epilogue_gate(result, row_scale, col_scale, bias, out_dtype)
        if vec4_ok:
            g.counters["vec4_epilogue"].hit()
            result = ops.epilogue_vec4(result, row_scale, col_scale)
        else:
            if g.vec4_epilogue_enabled:
                g.counters["vec4_epilogue"].refuse(
                    vec4_reason, result.shape, dtype=result.dtype,
                    contiguous=result.is_contiguous(), bias=bias is not None, out_dtype=out_dtype)
            g.counters["epilogue"].hit()
            result = ops.epilogue(result, row_scale, col_scale, fused_bias)
    else:
        g.counters["epilogue"].refuse("disabled" if not g.epilogue_enabled else "out_dtype",
                                      result.shape)
        result = g._fallback("epilogue")(result, row_scale, col_scale, bias, out_dtype)
    return result.reshape(*orig_shape[:-1], weight.shape[0])
