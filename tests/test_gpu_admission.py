"""Admission of every whitelisted production shape, element for element.

The reference admits an (M, K, N) into its launcher whitelist only after a full-shape
bitwise run of quantizer + GEMM + vec4-vs-scalar epilogue on the four DiT linears at that M
(validation/validate_conditioning_int8_shapes_hires.py:52-95 in the reference; the
whitelist comment at launcher/benchmark_launcher_v14_hires_int8_candidate.py:227 says every
listed shape is validated element for element) plus a round-half-even torture pattern per M
(:98-113 there).  This file is that harness for the per-rank token counts of the benchmark
configurations (4096; 23638 and 109099 tokens over 1/2/4/8 ranks) x the four linears of
the block.  Per shape, all at FULL size on the GPU:

  quantizer            vs the eager op sequence on the same device (q and scale bits)
  INT8 GEMM            vs torch._int_mm on the device (cuBLAS as the checker only)
  vec4 epilogue        vs the scalar epilogue
  fused GEMM+dequant   vs quantizer -> GEMM -> scalar epilogue with bias
  one-call linear      vs the same route
  64 sampled rows      vs the CPU oracle (q, scale bits, int32 accumulators, bf16 outputs)

and per M: the round-even pattern at K = 3072 and 8192, and swiglu-quant (the producer of
fc2's operand) vs the eager sequence on the same device.  Every comparison is an exact
mismatch COUNT that must be zero; the counts are printed per shape like the reference's
JSON report."""
import json

import pytest
import torch

from helpers import bits, tile_pattern

pytestmark = pytest.mark.gpu
DEV = "cuda:0"

# per-rank token counts of the benchmark configurations, as gates.LOCAL_M derives them
CONFIG_M = (4096, 23638, 11819, 5909, 5910, 2954, 2955, 109099, 54549, 54550, 27274, 27275, 13637, 13638)
# (K, N) of qkv, out-projection, fc1, fc2
LINEAR_KN = ((3072, 9216), (3072, 3072), (3072, 16384), (8192, 3072))
INV127 = 0.0078740157186985015869140625


def _count(a, b):
    return int(torch.count_nonzero(a != b).item())


def _eager_quantize(a):
    """The eager rowwise quantizer as an op sequence on the tensor's own device
    (kernels/exact-rowwise-int8/quantizer_kernel.hip:17-21 spells the order out)."""
    absmax = a.abs().amax(-1, keepdim=True)
    scale = (absmax.float() * INV127).clamp(min=1e-30)
    sm = scale.to(torch.bfloat16)
    sm = torch.where(sm == 0, torch.full_like(sm, 1.1754943508222875e-38), sm)
    r = (a / sm).float().round_()
    r.clamp_(-128.0, 127.0)          # rows with a NaN scale never occur in these inputs
    return r.to(torch.int8), scale


def _eager_swiglu_quantize(x):
    k = x.shape[1] // 2
    a = torch.nn.functional.silu(x[:, :k]) * x[:, k:]
    return _eager_quantize(a)


def test_config_m_is_what_the_gates_whitelist(pkg):
    gates = pkg.gates
    assert set(CONFIG_M) <= set(gates.LOCAL_M)
    for m in CONFIG_M:
        for k, n in LINEAR_KN:
            assert (m, k, n) in gates.GEMM_SHAPES
    derived = {4096} | {m for s in (23638, 109099) for p in (1, 2, 4, 8)
                        for m in pkg.ulysses.sequence_splits(s, p)}
    assert derived == set(CONFIG_M)


@pytest.mark.parametrize("m_index,m", list(enumerate(CONFIG_M)))
def test_admit_every_linear_at_this_token_count(cuda_pkg, ref, m_index, m):
    ops = cuda_pkg.ops
    report = []
    for shape_index, (k, n) in enumerate(LINEAR_KN):
        seed = 2026081200 + m_index * 100 + shape_index
        g = torch.Generator(device=DEV).manual_seed(seed)
        x = torch.randn((m, k), device=DEV, dtype=torch.bfloat16, generator=g)
        w = torch.randint(-127, 128, (n, k), device=DEV, dtype=torch.int8, generator=g)
        cs = (torch.rand((n,), device=DEV, dtype=torch.float32, generator=g) * 0.02 + 1e-5).contiguous()
        bias = torch.randn((n,), device=DEV, generator=g).to(torch.bfloat16)
        res = {"shape": [m, k, n]}

        q_ref, s_ref = _eager_quantize(x)
        q, s = ops.quantize_int8_rowwise(x)
        res["quantized_value_mismatch"] = _count(q_ref, q)
        res["quantized_scale_bit_mismatch"] = _count(bits(s_ref), bits(s))
        del q_ref, s_ref

        acc = ops.int_mm(q, w.t())
        acc_ref = torch._int_mm(q, w.t())
        res["int32_accumulator_mismatch"] = _count(acc_ref, acc)
        del acc_ref

        rs = s.reshape(-1).contiguous()
        scalar = ops.epilogue(acc, rs, cs, None)
        vec4 = ops.epilogue_vec4(acc, rs, cs)
        res["vec4_epilogue_bf16_mismatch"] = _count(bits(scalar), bits(vec4))
        del scalar, vec4

        three = ops.epilogue(acc, rs, cs, bias)
        fused = ops.int8_gemm_dequant(q, rs, w, cs, bias)
        res["fused_gemm_dequant_bf16_mismatch"] = _count(bits(three), bits(fused))
        one_call = ops.int8_linear(x, w, cs, bias)
        res["one_call_linear_bf16_mismatch"] = _count(bits(three), bits(one_call))
        del fused, one_call

        # 64 rows spread over the whole M range (first, last and the 128/256-row tile edges
        # included) against the CPU oracle
        rows = torch.unique(torch.cat((torch.tensor([0, 1, 127, 128, 255, 256, m - 2, m - 1]).clamp(0, m - 1),
                                       torch.linspace(0, m - 1, 56).long())))
        xr = x[rows.to(DEV)].cpu()
        q_cpu, s_cpu = ref.quantize_int8_rowwise(xr)
        acc_cpu = ref.int8_mm(q_cpu, w.cpu())
        out_cpu = ref.epilogue(acc_cpu, s_cpu.view(-1), cs.cpu(), bias.cpu())
        rd = rows.to(DEV)
        res["oracle_rows"] = int(rows.numel())
        res["oracle_q_mismatch"] = _count(q_cpu, q[rd].cpu())
        res["oracle_scale_bit_mismatch"] = _count(bits(s_cpu), bits(s[rd].cpu()))
        res["oracle_accumulator_mismatch"] = _count(acc_cpu, acc[rd].cpu())
        res["oracle_bf16_mismatch"] = _count(bits(out_cpu), bits(three[rd].cpu()))
        del acc, three, x, w
        report.append(res)
    ops.check_device_status()
    torch.cuda.empty_cache()
    print(json.dumps(report))
    for res in report:
        bad = {key: v for key, v in res.items() if key.endswith("mismatch") and v != 0}
        assert not bad, res


@pytest.mark.parametrize("m", CONFIG_M)
def test_round_even_pattern_and_swiglu_at_this_token_count(cuda_pkg, m):
    """The reference's per-M torture pattern (scale exactly 0.5: every .25/.75 is a tie
    after the division), at both quantizer widths, and the fused swiglu-quant at the FFN
    width; all against the eager sequence on the same device."""
    ops = cuda_pkg.ops
    report = []
    for k in (3072, 8192):
        x = tile_pattern([63.5, -63.5, 62.5, 1.25, 0.75, 0.25, -0.25, -0.75, -1.25, 0.0], m, k).to(DEV)
        q_ref, s_ref = _eager_quantize(x)
        q, s = ops.quantize_int8_rowwise(x)
        report.append({"shape": [m, k], "quantized_value_mismatch": _count(q_ref, q),
                       "quantized_scale_bit_mismatch": _count(bits(s_ref), bits(s))})
        del x, q_ref, s_ref, q, s
    g = torch.Generator(device=DEV).manual_seed(2026081300 + m)
    x = torch.randn((m, 16384), device=DEV, dtype=torch.bfloat16, generator=g)
    q_ref, s_ref = _eager_swiglu_quantize(x)
    q, s = ops.swiglu_quantize_int8_rowwise(x)
    report.append({"shape": [m, 16384], "op": "swiglu_quant", "quantized_value_mismatch": _count(q_ref, q),
                   "quantized_scale_bit_mismatch": _count(bits(s_ref), bits(s))})
    del x, q_ref, s_ref, q, s
    ops.check_device_status()
    torch.cuda.empty_cache()
    print(json.dumps(report))
    for res in report:
        assert res["quantized_value_mismatch"] == 0 and res["quantized_scale_bit_mismatch"] == 0, res
