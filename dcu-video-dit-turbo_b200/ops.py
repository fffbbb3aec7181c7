"""Torch-facing callables with the reference extensions' names and signatures.

Each function performs the argument checks of the reference's extension entry
point (raising RuntimeError as its TORCH_CHECKs do), allocates the outputs with
torch (the C library never allocates), and makes one C-ABI call that enqueues the
kernel on PyTorch's current stream.  Reference entry points, by path within the
reference project:

  quantize_int8_rowwise         kernels/exact-rowwise-int8/quantizer_kernel.hip:108-144
  epilogue                      kernels/int8-epilogue/epilogue_kernel.hip:65-133
  epilogue_vec4                 kernels/int8-epilogue-vec4/epilogue_kernel.hip:33-48
  mod_scale_shift_              kernels/mod-scale-shift/mod_kernel.hip:24-38
  swiglu_quantize_int8_rowwise  kernels/swiglu-quant/swiglu_quant_kernel.hip:111-137
  fwd_bhsd                      kernels/flash-attention-gfx936/csrc/flash_attn_hipc/h3_flash_api.cpp:30-130
  int_mm                        torch._int_mm call, launcher/benchmark_launcher_v14_hires_int8_candidate.py:823
"""
from __future__ import annotations

import math

import torch

from . import _lib

BIAS_NONE, BIAS_BF16, BIAS_FP32 = 0, 1, 2
ACT_NONE, ACT_SWIGLU = 0, 1

# kernels launched through this module since import (the benchmark's launch count)
launch_count = 0


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


class LaunchTimer:
    """CUDA events around every C-ABI launch made while the context is active.

        with ops.LaunchTimer() as timer:
            block.forward(x, cos, sin)
        for rec in timer.results(): ...   # {"name", "ms", "bound", "work"}

    `bound` names the roofline that limits the kernel ("hbm", "int8" or "bf16") and `work`
    its algorithmic bytes (hbm) or operations per launch, so a caller can turn `ms` into
    GB/s or TOP/s.  Events are recorded on PyTorch's current stream of the tensor's device
    (the stream the kernel is enqueued on); nothing synchronises until `results()`."""

    def __init__(self):
        self._records = []

    def __enter__(self):
        global _timer
        self._previous, _timer = _timer, self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = self._previous
        return False

    def results(self) -> list[dict]:
        out = []
        for name, e0, e1, work in self._records:
            e1.synchronize()
            bound, amount = work if work is not None else (None, None)
            out.append({"name": name, "ms": e0.elapsed_time(e1), "bound": bound, "work": amount})
        return out


_timer: LaunchTimer | None = None


def _call(name: str, t: torch.Tensor, *args, launches: int = 1, work=None) -> None:
    global launch_count
    lib = _lib.load()
    timer = _timer
    if timer is not None:
        stream = torch.cuda.current_stream(t.device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
    if t.device.index != torch.cuda.current_device():
        with torch.cuda.device(t.device):
            st = getattr(lib, name)(*args)
    else:
        st = getattr(lib, name)(*args)
    _lib.check(st, name)
    if timer is not None:
        e1.record(stream)
        timer._records.append((name, e0, e1, work))
    launch_count += launches


def _require_vector(v: torch.Tensor, like: torch.Tensor, numel: int, dtype, what: str) -> None:
    """A per-column operand handed to the C ABI as a raw pointer: right dtype, on the same
    CUDA device as the data, contiguous, with exactly `numel` elements."""
    _require(torch.is_tensor(v) and v.is_cuda and v.device == like.device,
             f"{what} must be on the same CUDA device as the data")
    _require(v.dtype == dtype, f"{what} must be {str(dtype).replace('torch.', '')}")
    _require(v.is_contiguous(), f"{what} must be contiguous")
    _require(v.numel() == numel, f"{what} must contain exactly {numel} values")


def quantize_int8_rowwise(x: torch.Tensor):
    """bf16 [M,K] -> [int8 [M,K], fp32 scale [M,1]], bit-identical to the eager op."""
    _require(x.is_cuda, "input must be on the CUDA device")
    _require(x.is_contiguous(), "input must be contiguous")
    _require(x.dtype == torch.bfloat16, "input must be bfloat16")
    _require(x.dim() == 2, "input must be a two-dimensional [M, K] tensor")
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=x.device)
    if m == 0:
        return [q, s]
    _call("b2_quantize_int8_rowwise", x, _ptr(x), _ptr(q), s.data_ptr(), m, k, _stream(x),
          work=("hbm", 3 * m * k + 4 * m))
    return [q, s]


def swiglu_quantize_int8_rowwise(x: torch.Tensor):
    """bf16 [M,2K] -> [int8 [M,K], fp32 [M,1]]: silu(gate)*up then the quantizer."""
    _require(x.is_cuda, "input must be on CUDA")
    _require(x.is_contiguous(), "input must be contiguous")
    _require(x.dtype == torch.bfloat16, "input must be BF16")
    _require(x.dim() == 2, "input must be [M, 2K]")
    _require(x.shape[1] % 2 == 0, "input width must be even")
    m, k = x.shape[0], x.shape[1] // 2
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=x.device)
    if m == 0 or k == 0:
        return [q, s]
    _call("b2_swiglu_quantize_int8_rowwise", x, x.data_ptr(), q.data_ptr(), s.data_ptr(), m, k,
          _stream(x), work=("hbm", 5 * m * k + 4 * m))
    return [q, s]


def _check_epilogue_common(acc, row_scale, col_scale):
    for t, name in ((acc, "accumulator"), (row_scale, "row_scale"), (col_scale, "col_scale")):
        _require(t.is_cuda, f"{name} must be on the CUDA device")
        _require(t.is_contiguous(), f"{name} must be contiguous")
    _require(acc.dtype == torch.int32, "accumulator must be int32")
    _require(row_scale.dtype == torch.float32, "row_scale must be float32")
    _require(col_scale.dtype == torch.float32, "col_scale must be float32")
    _require(acc.dim() == 2, "accumulator must be [M, N]")
    _require(row_scale.numel() == acc.shape[0], "row_scale must contain exactly M values")
    _require(col_scale.numel() == acc.shape[1], "col_scale must contain exactly N values")
    _require(row_scale.device == acc.device and col_scale.device == acc.device,
             "all inputs must be on the same device")


def _bias_kind(bias: torch.Tensor | None, n: int, device) -> int:
    if bias is None or bias.numel() == 0:
        return BIAS_NONE
    _require(bias.is_cuda and bias.device == device, "all inputs must be on the same device")
    _require(bias.is_contiguous(), "bias must be contiguous")
    _require(bias.numel() == n, "bias must be empty or contain exactly N values")
    if bias.dtype == torch.bfloat16:
        return BIAS_BF16
    if bias.dtype == torch.float32:
        return BIAS_FP32
    raise RuntimeError("bias must be empty, bfloat16, or float32")


def epilogue(acc: torch.Tensor, row_scale: torch.Tensor, col_scale: torch.Tensor,
             bias: torch.Tensor | None) -> torch.Tensor:
    """int32 [M,N] -> bf16 [M,N]; an empty (or None) bias means no bias."""
    _check_epilogue_common(acc, row_scale, col_scale)
    m, n = acc.shape
    kind = _bias_kind(bias, n, acc.device)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=acc.device)
    if acc.numel() == 0:
        return out
    _call("b2_epilogue", acc, acc.data_ptr(), row_scale.data_ptr(), col_scale.data_ptr(),
          _ptr(bias) if kind else None, kind, out.data_ptr(), m, n, _stream(acc),
          work=("hbm", 6 * m * n + 4 * m + 4 * n + (0, 2, 4)[kind] * n))
    return out


def epilogue_vec4(acc: torch.Tensor, row: torch.Tensor, col: torch.Tensor) -> torch.Tensor:
    """Bias-less 4-wide contract of the same epilogue."""
    _require(acc.is_cuda and row.is_cuda and col.is_cuda, "CUDA tensors required")
    _require(acc.is_contiguous() and row.is_contiguous() and col.is_contiguous(),
             "contiguous required")
    _require(acc.dtype == torch.int32 and row.dtype == torch.float32 and col.dtype == torch.float32,
             "dtype mismatch")
    _require(acc.dim() == 2 and row.numel() == acc.shape[0] and col.numel() == acc.shape[1],
             "shape mismatch")
    m, n = acc.shape
    out = torch.empty((m, n), dtype=torch.bfloat16, device=acc.device)
    if acc.numel() == 0:
        return out
    _call("b2_epilogue_vec4", acc, acc.data_ptr(), row.data_ptr(), col.data_ptr(), out.data_ptr(),
          m, n, _stream(acc), work=("hbm", 6 * m * n + 4 * m + 4 * n))
    return out


def mod_scale_shift_(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor) -> torch.Tensor:
    """In place x = bf16(bf16(x*bf16(1+scale)) + shift); returns x."""
    _require(x.is_cuda and scale.is_cuda and shift.is_cuda, "CUDA tensors required")
    _require(scale.device == x.device and shift.device == x.device,
             "all inputs must be on the same device")
    _require(x.is_contiguous() and scale.is_contiguous() and shift.is_contiguous(),
             "contiguous tensors required")
    _require(x.dtype == torch.bfloat16 and scale.dtype == torch.bfloat16
             and shift.dtype == torch.bfloat16, "BF16 required")
    _require(x.dim() == 2 and scale.numel() == x.shape[1] and shift.numel() == x.shape[1],
             "shape mismatch")
    if x.numel() == 0:
        return x
    _call("b2_mod_scale_shift", x, x.data_ptr(), scale.data_ptr(), shift.data_ptr(), x.shape[0],
          x.shape[1], _stream(x), work=("hbm", 4 * x.numel() + 4 * x.shape[1]))
    return x


def int_mm(a: torch.Tensor, w_t: torch.Tensor) -> torch.Tensor:
    """int32 [M,N] = a[M,K] @ w_t[K,N], with w_t the transpose VIEW of a contiguous
    int8 [N,K] weight: the same operands `torch._int_mm(x_8, weight.T)` receives."""
    _require(a.is_cuda and w_t.is_cuda, "CUDA tensors required")
    _require(a.device == w_t.device, "all inputs must be on the same device")
    _require(a.dtype == torch.int8 and w_t.dtype == torch.int8, "int8 operands required")
    _require(a.dim() == 2 and w_t.dim() == 2 and a.shape[1] == w_t.shape[0], "shape mismatch")
    _require(a.is_contiguous(), "a must be contiguous")
    w = w_t.t()
    _require(w.is_contiguous(), "w_t must be the transpose view of a contiguous [N,K] weight")
    m, k = a.shape
    n = w.shape[0]
    out = torch.empty((m, n), dtype=torch.int32, device=a.device)
    if m == 0 or n == 0:
        return out
    _call("b2_int8_gemm", a, a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, _stream(a),
          work=("int8", 2 * m * n * k))
    return out


def int8_gemm_dequant(a: torch.Tensor, row_scale: torch.Tensor, w: torch.Tensor,
                      col_scale: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
    """GEMM with the dequant epilogue fused: a int8 [M,K], w int8 [N,K] -> bf16 [M,N]."""
    _require(a.is_cuda and w.is_cuda and row_scale.is_cuda and col_scale.is_cuda,
             "CUDA tensors required")
    _require(w.device == a.device and row_scale.device == a.device and col_scale.device == a.device,
             "all inputs must be on the same device")
    _require(a.dtype == torch.int8 and w.dtype == torch.int8, "int8 operands required")
    _require(row_scale.dtype == torch.float32 and col_scale.dtype == torch.float32,
             "scales must be float32")
    _require(a.is_contiguous() and w.is_contiguous() and row_scale.is_contiguous()
             and col_scale.is_contiguous(), "contiguous required")
    _require(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "shape mismatch")
    m, k = a.shape
    n = w.shape[0]
    _require(row_scale.numel() == m and col_scale.numel() == n, "scale shape mismatch")
    kind = _bias_kind(bias, n, a.device)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=a.device)
    if m == 0 or n == 0:
        return out
    _call("b2_int8_gemm_dequant", a, a.data_ptr(), row_scale.data_ptr(), w.data_ptr(),
          col_scale.data_ptr(), _ptr(bias) if kind else None, kind, out.data_ptr(), m, n, k,
          _stream(a), work=("int8", 2 * m * n * k))
    return out


def int8_gemm_dequant_residual_(x: torch.Tensor, gate: torch.Tensor, a: torch.Tensor,
                                row_scale: torch.Tensor, w: torch.Tensor, col_scale: torch.Tensor,
                                bias: torch.Tensor | None) -> torch.Tensor:
    """x += gate * dequant(a @ w.T) with the block's roundings, in place on x bf16 [M,N]:
    the GEMM, its dequant epilogue and the gated residual in one kernel.  Returns x."""
    _require(a.is_cuda and a.dtype == torch.int8 and w.dtype == torch.int8 and a.is_contiguous()
             and w.is_contiguous() and a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1],
             "a int8 [M,K] and w int8 [N,K] must be contiguous CUDA tensors")
    m, k = a.shape
    n = w.shape[0]
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and tuple(x.shape) == (m, n),
             "x must be a contiguous CUDA bf16 [M,N] tensor")
    _require_vector(gate, a, n, torch.bfloat16, "gate")
    _require(w.is_cuda and w.device == a.device and x.device == a.device
             and row_scale.is_cuda and row_scale.device == a.device
             and col_scale.is_cuda and col_scale.device == a.device,
             "all inputs must be on the same device")
    _require(row_scale.dtype == torch.float32 and col_scale.dtype == torch.float32
             and row_scale.numel() == m and col_scale.numel() == n
             and row_scale.is_contiguous() and col_scale.is_contiguous(), "scale mismatch")
    kind = _bias_kind(bias, n, a.device)
    if m and n:
        _call("b2_int8_gemm_dequant_residual", a, a.data_ptr(), row_scale.data_ptr(), w.data_ptr(),
              col_scale.data_ptr(), _ptr(bias) if kind else None, kind, gate.data_ptr(),
              x.data_ptr(), m, n, k, _stream(a), work=("int8", 2 * m * n * k))
    return x


SWIGLU_GROUP = 64   # gate / up rows alternate in groups of this many in an interleaved projection


def interleave_gate_up(t: torch.Tensor, group: int = SWIGLU_GROUP) -> torch.Tensor:
    """Reorder the leading dimension of a SwiGLU projection's weight [2F, K], column scale [2F]
    or bias [2F] from (all gate rows, all up rows) to groups of `group` gate rows followed by
    the matching `group` up rows: the layout int8_gemm_dequant_swiglu reads.  Done once when
    the weights are loaded."""
    two_f = t.shape[0]
    _require(two_f % (2 * group) == 0, f"leading dimension must be a multiple of {2 * group}")
    f = two_f // 2
    gate, up = t[:f], t[f:]
    rest = tuple(t.shape[1:])
    return torch.stack((gate.reshape(f // group, group, *rest), up.reshape(f // group, group, *rest)),
                       dim=1).reshape(two_f, *rest).contiguous()


def int8_gemm_dequant_swiglu(a: torch.Tensor, row_scale: torch.Tensor, w_interleaved: torch.Tensor,
                             col_scale_interleaved: torch.Tensor,
                             bias_interleaved: torch.Tensor | None) -> torch.Tensor:
    """The FFN's first projection with SwiGLU in the GEMM's epilogue: returns
    bf16 [M, F] = bf16(bf16(silu(gate)) * up) of the dequantised projection, the operands
    interleaved by `interleave_gate_up`.  quantize_int8_rowwise of the result equals
    swiglu_quantize_int8_rowwise of the plain projection bit for bit."""
    _require(a.is_cuda and a.dtype == torch.int8 and w_interleaved.dtype == torch.int8 and a.is_contiguous()
             and w_interleaved.is_contiguous() and a.dim() == 2 and w_interleaved.dim() == 2
             and a.shape[1] == w_interleaved.shape[1],
             "a int8 [M,K] and w int8 [2F,K] must be contiguous CUDA tensors")
    m, k = a.shape
    n = w_interleaved.shape[0]
    _require(n % (2 * SWIGLU_GROUP) == 0, f"the projection width must be a multiple of {2 * SWIGLU_GROUP}")
    _require(w_interleaved.is_cuda and w_interleaved.device == a.device
             and row_scale.is_cuda and row_scale.device == a.device
             and col_scale_interleaved.is_cuda and col_scale_interleaved.device == a.device,
             "all inputs must be on the same device")
    _require(row_scale.dtype == torch.float32 and col_scale_interleaved.dtype == torch.float32
             and row_scale.numel() == m and col_scale_interleaved.numel() == n
             and row_scale.is_contiguous() and col_scale_interleaved.is_contiguous(), "scale mismatch")
    kind = _bias_kind(bias_interleaved, n, a.device)
    out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=a.device)
    if m and n:
        _call("b2_int8_gemm_dequant_swiglu", a, a.data_ptr(), row_scale.data_ptr(), w_interleaved.data_ptr(),
              col_scale_interleaved.data_ptr(), _ptr(bias_interleaved) if kind else None, kind,
              out.data_ptr(), m, n, k, _stream(a), work=("int8", 2 * m * n * k))
    return out


def int8_linear(x: torch.Tensor, w: torch.Tensor, col_scale: torch.Tensor,
                bias: torch.Tensor | None = None, input_act: str | None = None,
                scratch: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """One C call for (activation) -> quantize -> GEMM -> dequant.  x bf16 [M,K] (or
    [M,2K] with input_act="swiglu"); w int8 [N,K]; col_scale fp32 [N]."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous(),
             "x must be a contiguous CUDA bf16 [M,K] tensor")
    _require(w.is_cuda and w.dtype == torch.int8 and w.dim() == 2 and w.is_contiguous(),
             "w must be a contiguous CUDA int8 [N,K] tensor")
    act = {None: ACT_NONE, "swiglu": ACT_SWIGLU}.get(input_act, -1)
    _require(act >= 0, f"unknown input activation {input_act!r}")
    _require(act != ACT_SWIGLU or x.shape[1] % 2 == 0, "swiglu input width must be even")
    _require(w.device == x.device and col_scale.is_cuda and col_scale.device == x.device,
             "all inputs must be on the same device")
    m = x.shape[0]
    k = x.shape[1] // 2 if act == ACT_SWIGLU else x.shape[1]
    n = w.shape[0]
    if k != w.shape[1]:
        raise ValueError(
            f"Input and weight inner dimensions must match, got {k} and {w.shape[1]}")
    _require(col_scale.dtype == torch.float32 and col_scale.numel() == n
             and col_scale.is_contiguous(), "col_scale must be contiguous float32 [N]")
    kind = _bias_kind(bias, n, x.device)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    if m == 0 or n == 0:
        return out
    if scratch is None:
        qs = torch.empty((m, k), dtype=torch.int8, device=x.device)
        ss = torch.empty((m,), dtype=torch.float32, device=x.device)
    else:
        qs, ss = scratch
        _require(qs.numel() >= m * k and ss.numel() >= m, "scratch too small")
    _call("b2_int8_linear", x, x.data_ptr(), act, w.data_ptr(), col_scale.data_ptr(),
          _ptr(bias) if kind else None, kind, out.data_ptr(), qs.data_ptr(), ss.data_ptr(), m, n,
          k, _stream(x), launches=2, work=("int8", 2 * m * n * k))
    return out


def fwd_bhsd(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float) -> torch.Tensor:
    """bf16 FlashAttention forward on logical [B,H,S,128] inputs (any 16-byte-aligned
    strides with a contiguous last dimension).  Returns the [B,H,S,128] transpose
    VIEW of a fresh contiguous [B,S,H,128] tensor, so the caller's
    `.transpose(1,2).flatten(2)` is free."""
    _require(q.is_cuda and k.is_cuda and v.is_cuda, "q, k, and v must be on a CUDA device")
    _require(q.dtype == torch.bfloat16, "kernel requires BF16 q")
    _require(k.dtype == q.dtype and v.dtype == q.dtype, "q, k, and v must have the same dtype")
    _require(q.dim() == 4 and k.dim() == 4 and v.dim() == 4, "q, k, and v must use BHSD layout")
    _require(q.shape == k.shape and q.shape == v.shape,
             "kernel currently requires self-attention with identical QKV shapes")
    _require(q.device == k.device and q.device == v.device,
             "q, k, and v must be on the same CUDA device")
    _require(q.shape[3] == 128, "kernel requires head dimension 128")
    _require(q.stride(3) == 1 and k.stride(3) == 1 and v.stride(3) == 1,
             "q, k, and v must have contiguous last dimensions")
    _require(q.shape[0] > 0 and q.shape[1] > 0 and q.shape[2] > 0,
             "batch, heads, and sequence length must be positive")
    scale = float(softmax_scale)
    _require(math.isfinite(scale) and scale > 0.0, "softmax_scale must be finite and positive")
    b, h, s, d = q.shape
    storage = torch.empty((b, s, h, d), dtype=q.dtype, device=q.device)
    out = storage.transpose(1, 2)
    strides = []
    for t in (q, k, v):
        strides += [t.stride(0) if b > 1 else 0, t.stride(1) if h > 1 else 0, t.stride(2)]
    _call("b2_flash_fwd", q, q.data_ptr(), k.data_ptr(), v.data_ptr(), storage.data_ptr(), b, h, s,
          *strides, scale, _stream(q), work=("bf16", 4 * b * h * s * s * d))
    return out


# ---- DiT-block glue (no reference source; this package's own conventions) -------

def layernorm_mod(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor,
                  eps: float = 1e-6) -> torch.Tensor:
    """bf16 [M,C]: LayerNorm without affine, then the mod-scale-shift contract."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous(),
             "x must be a contiguous CUDA bf16 [M,C] tensor")
    _require_vector(scale, x, x.shape[1], torch.bfloat16, "scale")
    _require_vector(shift, x, x.shape[1], torch.bfloat16, "shift")
    out = torch.empty_like(x)
    if x.numel():
        _call("b2_layernorm_mod", x, x.data_ptr(), scale.data_ptr(), shift.data_ptr(),
              out.data_ptr(), x.shape[0], x.shape[1], eps, _stream(x), work=("hbm", 4 * x.numel()))
    return out


def layernorm_mod_quant(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor,
                        eps: float = 1e-6):
    """LayerNorm + modulation + rowwise quantizer in one pass: [int8 [M,C], fp32 [M,1]]."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous(),
             "x must be a contiguous CUDA bf16 [M,C] tensor")
    _require_vector(scale, x, x.shape[1], torch.bfloat16, "scale")
    _require_vector(shift, x, x.shape[1], torch.bfloat16, "shift")
    m, c = x.shape
    q = torch.empty((m, c), dtype=torch.int8, device=x.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=x.device)
    if x.numel():
        _call("b2_layernorm_mod_quant", x, x.data_ptr(), scale.data_ptr(), shift.data_ptr(),
              q.data_ptr(), s.data_ptr(), m, c, eps, _stream(x), work=("hbm", 3 * m * c + 4 * m))
    return [q, s]


def qk_norm_rope_(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                  cos: torch.Tensor, sin: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """In place on packed qkv bf16 [S,3,H,128]: per-head RMSNorm + rotary on q and k."""
    _require(qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 4
             and qkv.is_contiguous() and qkv.shape[1] == 3 and qkv.shape[3] == 128,
             "qkv must be a contiguous CUDA bf16 [S,3,H,128] tensor")
    s, _, h, _ = qkv.shape
    _require(tuple(cos.shape) == (s, 64) and tuple(sin.shape) == (s, 64), "cos/sin must be fp32 [S,64]")
    _require_vector(cos, qkv, s * 64, torch.float32, "cos")
    _require_vector(sin, qkv, s * 64, torch.float32, "sin")
    _require_vector(q_weight, qkv, 128, torch.bfloat16, "q norm weight")
    _require_vector(k_weight, qkv, 128, torch.bfloat16, "k norm weight")
    if s:
        _call("b2_qk_norm_rope", qkv, qkv.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr(),
              cos.data_ptr(), sin.data_ptr(), s, h, eps, _stream(qkv),
              work=("hbm", 8 * s * h * 128 + 512 * s))
    return qkv


def qk_norm_rope_pack(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                      cos: torch.Tensor, sin: torch.Tensor, world: int, chunks: int = 1,
                      eps: float = 1e-6) -> torch.Tensor:
    """qk_norm_rope_ fused with the pack of the sequence-parallel all-to-all: reads packed
    qkv bf16 [L,3,H,128] (left untouched) and returns the send buffer
    [chunks, world, L, c, 3, 128], c = H/(world*chunks); slice [ch] is one all-to-all."""
    _require(qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 4
             and qkv.is_contiguous() and qkv.shape[1] == 3 and qkv.shape[3] == 128,
             "qkv must be a contiguous CUDA bf16 [L,3,H,128] tensor")
    L, _, h, _ = qkv.shape
    _require(world > 0 and chunks > 0 and h % (world * chunks) == 0,
             "world*chunks must divide the head count")
    _require(tuple(cos.shape) == (L, 64) and tuple(sin.shape) == (L, 64), "cos/sin must be fp32 [L,64]")
    _require_vector(cos, qkv, L * 64, torch.float32, "cos")
    _require_vector(sin, qkv, L * 64, torch.float32, "sin")
    _require_vector(q_weight, qkv, 128, torch.bfloat16, "q norm weight")
    _require_vector(k_weight, qkv, 128, torch.bfloat16, "k norm weight")
    c = h // (world * chunks)
    send = torch.empty((chunks, world, L, c, 3, 128), dtype=torch.bfloat16, device=qkv.device)
    if L:
        _call("b2_qk_norm_rope_pack", qkv, qkv.data_ptr(), send.data_ptr(), q_weight.data_ptr(),
              k_weight.data_ptr(), cos.data_ptr(), sin.data_ptr(), L, h, world, chunks, eps,
              _stream(qkv), work=("hbm", 12 * L * h * 128 + 512 * L))
    return send


def qk_norm_rope_scatter(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                         cos: torch.Tensor, sin: torch.Tensor, recv_table, world: int, row0: int,
                         sequence: int, chunks: int = 1, eps: float = 1e-6) -> None:
    """qk_norm_rope_pack with the exchange folded in: every (head, part) of this rank's rows
    is stored straight into the receive buffer bf16 [chunks, S, c, 3, 128] of the rank that
    owns the head, at row `row0 + l`.  `recv_table` is a C array of `world` device addresses
    (peer.PeerBuffer.table).  Nothing waits: the caller orders the ranks (peer.PeerExchange)."""
    _require(qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 4
             and qkv.is_contiguous() and qkv.shape[1] == 3 and qkv.shape[3] == 128,
             "qkv must be a contiguous CUDA bf16 [L,3,H,128] tensor")
    L, _, h, _ = qkv.shape
    _require(0 < world <= 8 and chunks > 0 and h % (world * chunks) == 0,
             "world*chunks must divide the head count, with at most 8 ranks")
    _require(len(recv_table) == world, "one receive buffer per rank")
    _require(0 <= row0 and row0 + L <= sequence, "this rank's rows must lie inside the sequence")
    _require(tuple(cos.shape) == (L, 64) and tuple(sin.shape) == (L, 64), "cos/sin must be fp32 [L,64]")
    _require_vector(cos, qkv, L * 64, torch.float32, "cos")
    _require_vector(sin, qkv, L * 64, torch.float32, "sin")
    _require_vector(q_weight, qkv, 128, torch.bfloat16, "q norm weight")
    _require_vector(k_weight, qkv, 128, torch.bfloat16, "k norm weight")
    if L:
        _call("b2_qk_norm_rope_scatter", qkv, qkv.data_ptr(), recv_table, q_weight.data_ptr(),
              k_weight.data_ptr(), cos.data_ptr(), sin.data_ptr(), L, h, world, chunks, row0, sequence,
              eps, _stream(qkv),
              work=("nvlink", 6 * L * h * 128 * (world - 1) // world) if world > 1
              else ("hbm", 12 * L * h * 128 + 512 * L))


def copy_segments(src: torch.Tensor, src_offsets, src_table, dst_table, bytes_table, n: int,
                  total_bytes: int, remote_bytes: int = 0) -> None:
    """One launch copying n <= 8 contiguous byte ranges of `src` (at `src_offsets`, bytes) to
    the device addresses in `dst_table` (local or peer-mapped); the tables are C arrays,
    `src_table` is scratch that this call fills.  `remote_bytes` (of `total_bytes`) go to other
    GPUs: when non-zero the launch is accounted against the link, not against local memory."""
    _require(src.is_cuda and src.is_contiguous(), "source must be a contiguous CUDA tensor")
    _require(0 <= n <= 8 and len(src_offsets) == n, "at most 8 segments")
    base = src.data_ptr()
    limit = src.numel() * src.element_size()
    for i in range(n):
        _require(0 <= src_offsets[i] and src_offsets[i] + bytes_table[i] <= limit,
                 "a segment reaches outside the source tensor")
        src_table[i] = base + src_offsets[i]
    if n and total_bytes:
        _call("b2_copy_segments", src, src_table, dst_table, bytes_table, n, _stream(src),
              work=("nvlink", remote_bytes) if remote_bytes else ("hbm", 2 * total_bytes))


def quantize_int8_rowwise_gathered(x: torch.Tensor):
    """The rowwise quantizer reading the reverse all-to-all's receive buffer in place:
    x bf16 [chunks, world, M, w] (or [chunks, world, M, c, D]) holds row m's columns ((p*chunks + ch)*w ...) in segment
    (ch, p).  Returns [int8 [M, K], fp32 [M,1]] with K = chunks*world*w, identical to
    quantize_int8_rowwise of the unpacked [M,K] tensor."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() in (4, 5) and x.is_contiguous(),
             "input must be a contiguous CUDA bf16 [chunks, world, M, w] (or [..., c, D]) tensor")
    if x.dim() == 5:
        x = x.view(x.shape[0], x.shape[1], x.shape[2], x.shape[3] * x.shape[4])
    chunks, world, m, w = x.shape
    k = chunks * world * w
    _require(w % 8 == 0 and 0 < k <= 16384, "segment width must be a multiple of 8 and K <= 16384")
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    s = torch.empty((m, 1), dtype=torch.float32, device=x.device)
    if m:
        _call("b2_quantize_int8_rowwise_gathered", x, x.data_ptr(), q.data_ptr(), s.data_ptr(), m, k,
              world, chunks, _stream(x), work=("hbm", 3 * m * k + 4 * m))
    return [q, s]


_FRAME_DTYPES = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}


def images_to_u8(images: torch.Tensor) -> torch.Tensor:
    """Decoded frames (any shape, fp32 / bf16 / fp16, values nominally in [0,1]) -> uint8 of
    the same shape: `(images * 255).clamp(0, 255).byte()` for the whole clip in one launch
    (NaN -> 0)."""
    _require(images.is_cuda and images.is_contiguous(), "images must be a contiguous CUDA tensor")
    _require(images.dtype in _FRAME_DTYPES, "images must be float32, bfloat16 or float16")
    out = torch.empty(images.shape, dtype=torch.uint8, device=images.device)
    if images.numel():
        _call("b2_images_to_u8", images, images.data_ptr(), _FRAME_DTYPES[images.dtype], out.data_ptr(),
              images.numel(), _stream(images),
              work=("hbm", images.numel() * (images.element_size() + 1)))
    return out


def gate_residual_(x: torch.Tensor, y: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """In place x = bf16(x + bf16(gate*y)); returns x."""
    _require(x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.is_contiguous()
             and y.is_cuda and y.device == x.device and y.is_contiguous() and y.shape == x.shape
             and y.dtype == torch.bfloat16,
             "x,y must be contiguous bf16 [M,C] tensors on the same CUDA device")
    _require_vector(gate, x, x.shape[1], torch.bfloat16, "gate")
    if x.numel():
        _call("b2_gate_residual", x, x.data_ptr(), y.data_ptr(), gate.data_ptr(), x.shape[0],
              x.shape[1], _stream(x), work=("hbm", 6 * x.numel()))
    return x


def check_device_status(device=None) -> None:
    """Synchronise and raise if a bounded device-side wait gave up (on `device`, default:
    the current device; the status word lives in each device's copy of the library image)."""
    lib = _lib.load()
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(lib.b2_check_device_status(stream), "b2_check_device_status")
