"""CPU oracle for the DiT hot path: TEST INFRASTRUCTURE, not product code.

A plain PyTorch (CPU, eager) restatement of the reference's operators, one
function per operator, each written in the reference's exact operation order so
that results are bit-identical to the reference's own PyTorch implementation
(comfy-kitchen 0.2.26 eager ops, which are not part of the reference tree; the
reference's HIP kernels were each proven bit-identical to them and spell the
operation order out in comments).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module.  The product package never does: it fails loudly when its CUDA
library is missing.

Parity status: quantizer / epilogue / swiglu-quant / attention / Ulysses layout
are pinned by the reference's own in-tree generators and hand-derivable
known-answer vectors (tests/golden); mod-scale-shift is pinned only by the
kernel's comment; the DiT-block glue (LayerNorm, QK RMSNorm, RoPE, gating) has no
reference source at all and is "parity unpinned".
"""
from __future__ import annotations

import math

import torch

# fp32(1/127): ATen's GPU elementwise kernel strength-reduces `/ 127.0` into a
# multiply by this constant (kernels/exact-rowwise-int8/quantizer_kernel.hip:68-73).
# PyTorch-CPU would do a true division, which differs for 1488 bf16 maxima, so the
# multiply is spelled out.
INV127 = 0.0078740157186985015869140625
SCALE_FLOOR = 1.0e-30
BF16_TINY = 1.1754943508222875e-38


def _quantize_with_absmax(values: torch.Tensor, abs_max: torch.Tensor):
    """Scale + quantise step shared by the quantizer and swiglu-quant.

    kernels/exact-rowwise-int8/quantizer_kernel.hip:17-21 (operation order),
    :72-83 (scale floor, bf16 scale, zero replacement), :92-104 (bf16 division,
    round-half-even, clamp [-128,127], non-finite -> 0).
    """
    scale = abs_max.float() * torch.tensor(INV127, dtype=torch.float32)
    # clamp(min=...) keeps NaN, exactly like the kernel's `!isnan(scale) &&` guard
    scale = scale.clamp(min=SCALE_FLOOR)
    scale_math = scale.to(torch.bfloat16)
    tiny = torch.tensor(BF16_TINY, dtype=torch.float32).to(torch.bfloat16)
    scale_math = torch.where(scale_math == 0, tiny, scale_math)
    divided = values / scale_math  # fp32 divide, rounded to bf16
    rounded = divided.float().round()  # ties to even
    rounded = torch.where(rounded > 127.0, torch.full_like(rounded, 127.0), rounded)
    rounded = torch.where(rounded < -128.0, torch.full_like(rounded, -128.0), rounded)
    finite = torch.isfinite(rounded)
    q = torch.where(finite, rounded, torch.zeros_like(rounded)).to(torch.int8)
    return q, scale


def quantize_int8_rowwise(x: torch.Tensor):
    """bf16 [M,K] -> (int8 [M,K], fp32 scale [M,1]).

    kernels/exact-rowwise-int8/quantizer_kernel.hip:118-144; empty-input rules
    :124-129 (rows != 0 and K == 0 -> scales filled with 1e-30).
    """
    assert x.dtype == torch.bfloat16 and x.dim() == 2
    rows, cols = x.shape
    if x.numel() == 0:
        q = torch.empty((rows, cols), dtype=torch.int8)
        s = torch.empty((rows, 1), dtype=torch.float32)
        if rows != 0 and cols == 0:
            s.fill_(SCALE_FLOOR)
        return q, s
    abs_max = x.abs().amax(-1, keepdim=True)  # bf16, NaN-propagating
    return _quantize_with_absmax(x, abs_max)


def epilogue(acc: torch.Tensor, row_scale: torch.Tensor, col_scale: torch.Tensor,
             bias: torch.Tensor | None = None) -> torch.Tensor:
    """int32 [M,N] * (rs[m]*cs[n]) -> bf16, then optional + bf16(bias) -> bf16.

    kernels/int8-epilogue/epilogue_kernel.hip:39-53; eager transcription in
    kernels/int8-epilogue/bench.py:33-48 (same values: the chunking there only
    bounds temporaries).  A zero-element bias means "none" (:97-107).
    """
    assert acc.dtype == torch.int32 and acc.dim() == 2
    combined = row_scale.reshape(-1, 1).float() * col_scale.reshape(1, -1).float()
    out = (acc.float() * combined).to(torch.bfloat16)
    if bias is not None and bias.numel() != 0:
        b = bias.to(torch.bfloat16).reshape(1, -1)
        out = out + b  # fp32 add of two bf16, rounded to bf16
    return out


def mod_scale_shift(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    """bf16( bf16(x * bf16(1+scale)) + shift ), three bf16 roundings.

    kernels/mod-scale-shift/mod_kernel.hip:16-21.  Returns a new tensor (the
    product op works in place).
    """
    assert x.dtype == torch.bfloat16 and x.dim() == 2
    factor = (1.0 + scale.reshape(1, -1).float()).to(torch.bfloat16)
    product = (x.float() * factor.float()).to(torch.bfloat16)
    return (product.float() + shift.reshape(1, -1).float()).to(torch.bfloat16)


def swiglu(x: torch.Tensor) -> torch.Tensor:
    """bf16( bf16(silu_fp32(gate)) * up ), gate = first half of the row.

    kernels/swiglu-quant/swiglu_quant_kernel.hip:18-27,43-44.
    silu(g) = g / (1 + expf(-g)) in fp32.
    """
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 2 == 0
    k = x.shape[1] // 2
    gate = x[:, :k].float()
    up = x[:, k:].float()
    silu = (gate / (1.0 + torch.exp(-gate))).to(torch.bfloat16)
    return (silu.float() * up).to(torch.bfloat16)


def swiglu_quantize_int8_rowwise(x: torch.Tensor):
    """Fused SwiGLU + rowwise quantizer: bf16 [M,2K] -> (int8 [M,K], fp32 [M,1]).

    kernels/swiglu-quant/swiglu_quant_kernel.hip:111-137 (zero rows or zero
    columns return uninitialised outputs, :121-123).
    """
    rows = x.shape[0]
    k = x.shape[1] // 2
    if rows == 0 or k == 0:
        return (torch.empty((rows, k), dtype=torch.int8),
                torch.empty((rows, 1), dtype=torch.float32))
    a = swiglu(x)
    abs_max = a.abs().amax(-1, keepdim=True)
    return _quantize_with_absmax(a, abs_max)


def int8_mm(a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """acc[M,N] = A[M,K] . W[N,K]^T in exact int32.

    launcher/benchmark_launcher_v14_hires_int8_candidate.py:823
    (`torch._int_mm(x_8, weight.T)`).  Integers are exact, so any correct int32
    matmul is the oracle; CPU `torch._int_mm` needs M > 16, so small cases use an
    int64 matmul cast down.
    """
    assert a.dtype == torch.int8 and w.dtype == torch.int8
    if a.shape[0] > 16 and a.shape[0] % 8 == 0 and a.shape[1] % 8 == 0 and w.shape[0] % 8 == 0:
        try:
            return torch._int_mm(a, w.t())
        except RuntimeError:
            pass
    # float64 holds |acc| <= 128*128*K exactly for every K of interest
    return (a.double() @ w.double().t()).to(torch.int32)


def int8_linear(x: torch.Tensor, weight: torch.Tensor, weight_scale: torch.Tensor,
                bias: torch.Tensor | None = None, input_act: str | None = None) -> torch.Tensor:
    """activation -> quantize -> int8 GEMM -> dequant epilogue -> reshape.

    launcher/benchmark_launcher_v14_hires_int8_candidate.py:960-1067 (bf16 output,
    no ConvRot).  weight int8 [N,K]; weight_scale scalar or [N] (:986-991,
    :1011-1015).
    """
    if input_act == "swiglu":
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        q, s = swiglu_quantize_int8_rowwise(x2)
    else:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        q, s = quantize_int8_rowwise(x2)
    if q.shape[-1] != weight.shape[-1]:
        raise ValueError("Input and weight inner dimensions must match")
    ws = weight_scale.float().reshape(-1)
    if ws.numel() not in (1, weight.shape[0]):
        raise ValueError("INT8 weight scale must be scalar or per-output-channel")
    if ws.numel() == 1:
        ws = ws.expand(weight.shape[0]).contiguous()
    acc = int8_mm(q, weight)
    out = epilogue(acc, s.reshape(-1), ws, bias)
    return out.reshape(*lead, weight.shape[0])


def quantize_weight_per_channel(w: torch.Tensor):
    """Weight pre-quantisation used by the benchmark configs (no reference code;
    defined by the benchmark description): per output channel symmetric int8,
    scale = absmax/127 (fp32 true division), round-half-even, clamp +-127."""
    wf = w.float()
    scale = (wf.abs().amax(-1) / 127.0).clamp(min=1e-30)
    q = (wf / scale[:, None]).round().clamp(-127, 127).to(torch.int8)
    return q, scale


def attention_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                   row_chunk: int = 2048) -> torch.Tensor:
    """fp32 math attention on [B,H,S,D] inputs, chunked over query rows.

    validation/validate_flash_longseq.py:37-42 and
    benchmarks/bench_opendas_h3_flash_bshd.py:71-74.  Returns fp32 [B,H,S,D].
    """
    b, h, s, d = q.shape
    out = torch.empty((b, h, s, d), dtype=torch.float32)
    for bi in range(b):
        for hi in range(h):
            kf = k[bi, hi].float()
            vf = v[bi, hi].float()
            for r0 in range(0, s, row_chunk):
                r1 = min(s, r0 + row_chunk)
                scores = (q[bi, hi, r0:r1].float() @ kf.T) * scale
                out[bi, hi, r0:r1] = torch.softmax(scores, dim=-1) @ vf
    return out


def attention_rows_fp32(q, k, v, head: int, r0: int, r1: int, scale: float) -> torch.Tensor:
    """Sampled-rows fp32 reference, validation/validate_flash_longseq.py:37-42."""
    qf = q[0, head, r0:r1].float()
    kf = k[0, head].float()
    vf = v[0, head].float()
    return torch.softmax((qf @ kf.T) * scale, dim=-1) @ vf


# ----------------------------------------------------------------------------
# Ulysses layout transforms (single-process model of the all-to-all)
# ----------------------------------------------------------------------------

def ulysses_splits(seq: int, world: int) -> list[int]:
    """Token split: the first `seq % world` ranks hold one extra row."""
    base, rem = divmod(seq, world)
    return [base + (1 if r < rem else 0) for r in range(world)]


def sequence_to_heads_all(shards: list[torch.Tensor]) -> list[torch.Tensor]:
    """All ranks at once: token-sharded [L_r,H,D] -> head-sharded [S,H/P,D].

    benchmarks/bench_sp_head_chunk_overlap.py:83-98.
    """
    world = len(shards)
    h = shards[0].shape[1]
    hl = h // world
    full = torch.cat(shards, dim=0)
    return [full[:, r * hl:(r + 1) * hl].contiguous() for r in range(world)]


def heads_to_sequence_all(heads: list[torch.Tensor], splits: list[int]) -> list[torch.Tensor]:
    """Inverse: head-sharded [S,H/P,D] per rank -> token-sharded [L_r,H,D].

    benchmarks/bench_sp_head_chunk_overlap.py:100-118.
    """
    full = torch.cat(heads, dim=1)
    return [t.contiguous() for t in full.split(splits, dim=0)]


def pack_send(qkv: torch.Tensor, world: int, chunks: int) -> torch.Tensor:
    """Packed projection output [L,3,H,D] -> destination-major send buffer
    [chunks, world, L, c, 3, D], c = H/(world*chunks), head h = (p*chunks + ch)*c + ci.
    Slice [ch] is the [world, L, c, 3, D] buffer of
    benchmarks/bench_sp_head_chunk_overlap.py:140-164."""
    L, _, h, d = qkv.shape
    c = h // (world * chunks)
    return qkv.reshape(L, 3, world, chunks, c, d).permute(3, 2, 0, 4, 1, 5).contiguous()


def unpack_gathered(recv: torch.Tensor) -> torch.Tensor:
    """Reverse all-to-all receive buffer [chunks, world, L, c, D] -> [L, H*D] in head order
    h = (p*chunks + ch)*c + ci."""
    chunks, world, L, c, d = recv.shape
    return recv.permute(2, 1, 0, 3, 4).reshape(L, world * chunks * c * d).contiguous()


def images_to_u8(images: torch.Tensor) -> torch.Tensor:
    """`(images * 255).clamp(0, 255).byte()`, the expression the reference batches over a
    whole clip (launcher/benchmark_launcher_v14_hires_int8_candidate.py:645-647); the product
    keeps the input dtype, the cast truncates.  NaN (undefined in that cast) is defined as 0."""
    prod = images * 255
    prod = torch.where(torch.isnan(prod), torch.zeros_like(prod), prod)
    return prod.clamp(0, 255).to(torch.uint8)


# ----------------------------------------------------------------------------
# DiT block glue.  No reference source exists for these (they live in ComfyUI's
# model file, which is not part of the reference tree): PARITY UNPINNED.  The
# conventions below are this project's own, documented with the block.
# ----------------------------------------------------------------------------

def layer_norm_noaffine(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """fp32 LayerNorm without affine over the last dim, result rounded to bf16."""
    xf = x.float()
    mean = xf.mean(-1, keepdim=True)
    var = ((xf - mean) ** 2).mean(-1, keepdim=True)
    return ((xf - mean) * torch.rsqrt(var + eps)).to(torch.bfloat16)


def rope_tables(positions: torch.Tensor, head_dim: int = 128, axes=(32, 48, 48),
                theta: float = 10000.0):
    """3-D rotary tables: positions int [S,3] (t,y,x); the head dim is split into
    three axis bands of `axes` channels, each band rotating adjacent pairs
    (2i, 2i+1) with frequency theta^(-2i/band).  Returns cos,sin fp32 [S,D/2]."""
    assert sum(axes) == head_dim
    cos, sin = [], []
    for a, band in enumerate(axes):
        half = band // 2
        inv = theta ** (-torch.arange(half, dtype=torch.float64) * 2.0 / band)
        ang = positions[:, a].double()[:, None] * inv[None, :]
        cos.append(torch.cos(ang).float())
        sin.append(torch.sin(ang).float())
    return torch.cat(cos, -1).contiguous(), torch.cat(sin, -1).contiguous()


def qk_norm_rope(x: torch.Tensor, weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 eps: float = 1e-6) -> torch.Tensor:
    """Per-head RMSNorm (fp32, weight bf16 [D]) then rotary on adjacent pairs.

    x bf16 [S,H,D].  y = x * rsqrt(mean(x^2)+eps) * w (fp32, no intermediate
    rounding), then (y0*c - y1*s, y1*c + y0*s), rounded once to bf16."""
    xf = x.float()
    rms = torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
    y = xf * rms * weight.float()
    y0, y1 = y[..., 0::2], y[..., 1::2]
    c, s = cos[:, None, :], sin[:, None, :]
    o0 = y0 * c - y1 * s
    o1 = y1 * c + y0 * s
    return torch.stack((o0, o1), dim=-1).flatten(-2).to(torch.bfloat16)


def gate_residual(x: torch.Tensor, y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """x + gate*y with two bf16 roundings: bf16(x + bf16(gate*y))."""
    prod = (y.float() * gate.reshape(1, -1).float()).to(torch.bfloat16)
    return (x.float() + prod.float()).to(torch.bfloat16)


def dit_block(x: torch.Tensor, p: dict, cos: torch.Tensor, sin: torch.Tensor,
              heads: int = 24, head_dim: int = 128) -> torch.Tensor:
    """One DiT block (benchmark config 4), composed from the oracle ops.

    adaLN(shift,scale) -> INT8 qkv -> per-head QK RMSNorm + 3-D RoPE -> attention
    -> INT8 out-proj -> gated residual -> adaLN -> INT8 fc1 -> SwiGLU -> INT8 fc2
    -> gated residual.  `p` holds mod vectors (bf16 [C]) shift1, scale1, gate1,
    shift2, scale2, gate2; int8 weights wq_*, fp32 per-channel scales ws_*, bf16
    biases b_*; q_norm_w, k_norm_w bf16 [D].
    """
    s, c = x.shape
    h = mod_scale_shift(layer_norm_noaffine(x), p["scale1"], p["shift1"])
    qkv = int8_linear(h, p["wq_qkv"], p["ws_qkv"], p["b_qkv"])
    qkv = qkv.reshape(s, 3, heads, head_dim)
    q = qk_norm_rope(qkv[:, 0], p["q_norm_w"], cos, sin)
    k = qk_norm_rope(qkv[:, 1], p["k_norm_w"], cos, sin)
    v = qkv[:, 2]
    o = attention_fp32(q.transpose(0, 1)[None], k.transpose(0, 1)[None],
                       v.transpose(0, 1)[None], head_dim ** -0.5)
    o = o[0].transpose(0, 1).reshape(s, c).to(torch.bfloat16)
    a = int8_linear(o, p["wq_out"], p["ws_out"], p["b_out"])
    x = gate_residual(x, a, p["gate1"])
    h = mod_scale_shift(layer_norm_noaffine(x), p["scale2"], p["shift2"])
    f = int8_linear(h, p["wq_fc1"], p["ws_fc1"], p["b_fc1"])
    f = int8_linear(f, p["wq_fc2"], p["ws_fc2"], p["b_fc2"], input_act="swiglu")
    return gate_residual(x, f, p["gate2"])


def psnr(ref: torch.Tensor, got: torch.Tensor) -> float:
    """Peak signal-to-noise ratio in dB with the reference's peak-to-peak range."""
    r, g = ref.double(), got.double()
    mse = float(((r - g) ** 2).mean())
    if mse == 0.0:
        return math.inf
    peak = float(r.max() - r.min())
    return 10.0 * math.log10(peak * peak / mse)
