"""Exactness gates: shape whitelists, artifact audit, counted refusal with fallback.

Mirror of the gate layer in the reference's launcher
(launcher/benchmark_launcher_v14_hires_int8_candidate.py): every operator is
opt-in through an environment flag read at construction, hard-fails at start-up
when enabled but unloadable (:219-222, :936-948), is substituted only when its
complete contract matches, and otherwise is REFUSED with a reason string: the
refusal is counted, logged once per (reason, shape) and the call goes to the
host application's original implementation.  The order of the refusal reasons is
part of the interface (the reference asserts it one reason at a time in
kernels/int8-epilogue-vec4/verify_v11_contract.py:81-103).

Differences from the reference, all deliberate:
  * "arch" means compute capability 10.x (sm_100) instead of gfx936;
  * an "audit" reason follows "disabled": the loaded artifact's sha256 must be in
    the audit table (the reference paper's SUBSTITUTE rule, paper/draft.md:88-97,
    which its launcher only approximates with contract strings);
  * whitelists hold this deployment's shapes (hidden 3072, 24 heads, FFN 8192 and
    the per-rank token counts for 1/2/4/8 GPUs) next to the reference's own;
  * the log de-duplication key is (reason, shape) so each refused M is reported
    (the reference's reason-only key hid later refused M values);
  * fallbacks are supplied by the host (`register_fallbacks`); this package ships
    no eager implementation, and a refusal without a registered fallback raises.
"""
from __future__ import annotations

import atexit
import json
import logging
import os
from collections import Counter
from typing import Callable

import torch

from . import _lib, ops

log = logging.getLogger("b2dit.gates")


def _split(seq: int, world: int) -> tuple[int, ...]:
    base, rem = divmod(seq, world)
    return tuple(sorted({base, base + 1} if rem else {base}))


# Per-rank token counts: benchmark shapes (4096; 23638 and 109099 tokens over 1/2/4/8
# ranks) plus the reference's own local M values (launcher :111).
REFERENCE_LOCAL_M = (11819, 12055, 12280, 18873, 18874, 36711, 36712, 54549, 54550)
LOCAL_M = frozenset(
    {4096} | {m for s in (23638, 109099) for p in (1, 2, 4, 8) for m in _split(s, p)}
    | set(REFERENCE_LOCAL_M))
QUANTIZER_K = frozenset((3072, 8192, 5376, 7168, 14336))
SWIGLU_K = frozenset((8192, 14336))
MOD_C = frozenset((3072, 5376))
EPILOGUE_N = frozenset((3072, 9216, 16384, 5376, 21504, 28672))
# (K, N) of the four DiT linears: qkv, out, fc1, fc2 (launcher :229-245 analogues)
LINEAR_KN = frozenset(((3072, 9216), (3072, 3072), (3072, 16384), (8192, 3072),
                       (5376, 21504), (7168, 5376), (5376, 28672), (14336, 5376)))
GEMM_SHAPES = frozenset((m, k, n) for m in LOCAL_M for (k, n) in LINEAR_KN)
WEIGHT_SHAPES = frozenset((n, k) for (k, n) in LINEAR_KN)
FLASH_HEADS = frozenset((24, 12, 6, 3, 28, 14))
FLASH_HEAD_CHUNKS = frozenset((1, 2, 3, 4, 6, 8, 12, 14))
FLASH_MAX_SEQ = 131072
SP_WORLDS = frozenset((1, 2, 4, 8))


def _flag(name: str) -> bool:
    return os.environ.get(name, "0") == "1"


def is_sm100(tensor) -> bool:
    """Compute capability 10.x of the tensor's device (the `arch` condition)."""
    if not getattr(tensor, "is_cuda", False):
        return False
    try:
        return torch.cuda.get_device_capability(tensor.device)[0] == 10
    except (AttributeError, RuntimeError, AssertionError):
        return False


class GateCounters:
    """hits / fallbacks / reasons for one operator, with the reference's log cadence."""

    def __init__(self, name: str):
        self.name = name
        self.hits = 0
        self.fallbacks: Counter = Counter()
        self._logged: set = set()

    def hit(self) -> None:
        self.hits += 1
        if self.hits == 1 or self.hits % 500 == 0:
            log.warning("B200 %s hits=%d fallbacks=%d", self.name, self.hits,
                        sum(self.fallbacks.values()))

    def refuse(self, reason: str, shape, **detail) -> None:
        self.fallbacks[reason] += 1
        key = (reason, tuple(shape) if shape is not None else None)
        if key not in self._logged and len(self._logged) < 64:
            self._logged.add(key)
            log.warning("B200 %s fallback reason=%s shape=%s %s", self.name, reason, key[1],
                        " ".join(f"{k}={v}" for k, v in detail.items()))

    def summary(self) -> dict:
        return {"hits": self.hits, "fallbacks": sum(self.fallbacks.values()),
                "reasons": dict(sorted(self.fallbacks.items()))}


class Gates:
    """One configuration of the gate layer.  `Gates.from_env()` reads the reference's
    flag names (H3_INT8_EXACT_QUANTIZER, H3_INT8_EPILOGUE, H3_INT8_EPILOGUE_VEC4,
    H3_INT8_UNPADDED_M, H3_FLASH_ATTN, H3_SP_HEAD_CHUNK_OVERLAP; all default off)
    plus H3_MOD_SCALE_SHIFT, H3_SWIGLU_QUANT and H3_INT8_FUSED_GEMM for the operators
    the reference never wired into a launcher."""

    def __init__(self, *, exact_quantizer=False, epilogue=False, epilogue_vec4=False,
                 unpadded_m=False, flash=False, head_chunk_overlap=False, mod_scale_shift=False,
                 swiglu_quant=False, fused_gemm=False, sp_world: int = 1, load: bool = True):
        self.exact_quantizer_enabled = exact_quantizer
        self.epilogue_enabled = epilogue
        self.vec4_epilogue_enabled = epilogue_vec4
        self.unpadded_m_enabled = unpadded_m
        self.flash_enabled = flash
        self.head_chunk_overlap_enabled = head_chunk_overlap
        self.mod_scale_shift_enabled = mod_scale_shift
        self.swiglu_quant_enabled = swiglu_quant
        self.fused_gemm_enabled = fused_gemm
        self.sp_world = sp_world
        self.is_arch = is_sm100
        self.audited: Callable[[str], bool] = _lib.audited
        self.fallbacks: dict[str, Callable] = {}
        self.counters = {n: GateCounters(n) for n in
                         ("exact_quantizer", "vec4_epilogue", "epilogue", "unpadded_gemm",
                          "fused_gemm", "mod_scale_shift", "swiglu_quant", "flash", "convrot")}
        self.flash_fallback_signatures: set = set()
        self.flash_head_chunk_calls = 0
        self._flash_first_call = True
        # host hooks of the attention gate (None = the defaults in attention.py):
        # context_resolver(transformer_options) -> sequence-parallel context or None,
        # precision_resolver(attn_precision, dtype) -> the precision the host will really use
        self.context_resolver: Callable | None = None
        self.precision_resolver: Callable | None = None
        # start-up invariants (launcher :936-941): vec4 needs the scalar epilogue as
        # its fallback; any enabled feature needs a loadable artifact NOW.
        if self.vec4_epilogue_enabled and not self.epilogue_enabled:
            raise RuntimeError(
                "H3_INT8_EPILOGUE_VEC4=1 requires H3_INT8_EPILOGUE=1 so every ineligible call "
                "can fall back to the existing exact epilogue")
        if load and self.any_enabled():
            _lib.load()
            log.warning("B200 DiT kernels loaded: %s sha256=%s audited=%s", _lib.so_path(),
                        _lib.loaded_sha256()[:16], _lib.audited())

    @classmethod
    def from_env(cls, **overrides) -> "Gates":
        kw = dict(exact_quantizer=_flag("H3_INT8_EXACT_QUANTIZER"), epilogue=_flag("H3_INT8_EPILOGUE"),
                  epilogue_vec4=_flag("H3_INT8_EPILOGUE_VEC4"), unpadded_m=_flag("H3_INT8_UNPADDED_M"),
                  flash=_flag("H3_FLASH_ATTN"), head_chunk_overlap=_flag("H3_SP_HEAD_CHUNK_OVERLAP"),
                  mod_scale_shift=_flag("H3_MOD_SCALE_SHIFT"), swiglu_quant=_flag("H3_SWIGLU_QUANT"),
                  fused_gemm=_flag("H3_INT8_FUSED_GEMM"))
        kw.update(overrides)
        return cls(**kw)

    @classmethod
    def all_on(cls, **overrides) -> "Gates":
        kw = dict(exact_quantizer=True, epilogue=True, epilogue_vec4=True, unpadded_m=True,
                  flash=True, head_chunk_overlap=True, mod_scale_shift=True, swiglu_quant=True,
                  fused_gemm=True)
        kw.update(overrides)
        return cls(**kw)

    def any_enabled(self) -> bool:
        return any((self.exact_quantizer_enabled, self.epilogue_enabled, self.vec4_epilogue_enabled,
                    self.unpadded_m_enabled, self.flash_enabled, self.mod_scale_shift_enabled,
                    self.swiglu_quant_enabled, self.fused_gemm_enabled))

    def register_fallbacks(self, **fns: Callable) -> None:
        """Host-supplied original implementations: quantize, swiglu_quantize, int_mm,
        epilogue, mod_scale_shift, attention, input_act, convrot_rotate."""
        self.fallbacks.update(fns)

    def _fallback(self, name: str) -> Callable:
        fn = self.fallbacks.get(name)
        if fn is None:
            raise RuntimeError(f"B200 gate refused the call and no '{name}' fallback is registered")
        return fn

    # ---- gates: (eligible, reason) in the reference's order ----------------------
    def exact_quantizer_gate(self, x, stochastic_rounding: int = 0):
        """launcher :157-179."""
        if not self.exact_quantizer_enabled:
            return False, "disabled"
        if not self.audited("quantize_int8_rowwise"):
            return False, "audit"
        if stochastic_rounding != 0:
            return False, "stochastic_rounding"
        if x.dtype != torch.bfloat16:
            return False, "dtype"
        if not x.is_cuda:
            return False, "device"
        if x.requires_grad:
            return False, "requires_grad"
        if not x.is_contiguous():
            return False, "noncontiguous"
        if x.dim() != 2 or x.shape[0] not in LOCAL_M:
            return False, "M"
        if x.shape[1] not in QUANTIZER_K:
            return False, "K"
        if not self.is_arch(x):
            return False, "arch"
        return True, "eligible"

    def swiglu_quant_gate(self, x, stochastic_rounding: int = 0):
        """The quantizer's pattern applied to the fused SwiGLU input [M, 2K]."""
        if not self.swiglu_quant_enabled:
            return False, "disabled"
        if not self.audited("swiglu_quantize_int8_rowwise"):
            return False, "audit"
        if stochastic_rounding != 0:
            return False, "stochastic_rounding"
        if x.dtype != torch.bfloat16:
            return False, "dtype"
        if not x.is_cuda:
            return False, "device"
        if x.requires_grad:
            return False, "requires_grad"
        if not x.is_contiguous():
            return False, "noncontiguous"
        if x.dim() != 2 or x.shape[0] not in LOCAL_M:
            return False, "M"
        if x.shape[1] % 2 != 0 or x.shape[1] // 2 not in SWIGLU_K:
            return False, "K"
        if not self.is_arch(x):
            return False, "arch"
        return True, "eligible"

    def mod_scale_shift_gate(self, x, scale, shift):
        if not self.mod_scale_shift_enabled:
            return False, "disabled"
        if not self.audited("mod_scale_shift"):
            return False, "audit"
        if x.dtype != torch.bfloat16 or scale.dtype != torch.bfloat16 or shift.dtype != torch.bfloat16:
            return False, "dtype"
        if not (x.is_cuda and scale.is_cuda and shift.is_cuda):
            return False, "device"
        if x.requires_grad:
            return False, "requires_grad"
        if not (x.is_contiguous() and scale.is_contiguous() and shift.is_contiguous()):
            return False, "noncontiguous"
        if x.dim() != 2 or x.shape[0] not in LOCAL_M:
            return False, "M"
        if x.shape[1] not in MOD_C:
            return False, "C"
        if scale.numel() != x.shape[1] or shift.numel() != x.shape[1]:
            return False, "vector_shape"
        if not self.is_arch(x):
            return False, "arch"
        return True, "eligible"

    def vec4_epilogue_gate(self, accumulator, row_scale, col_scale, bias, out_dtype):
        """launcher :863-904, reason for reason."""
        if not self.vec4_epilogue_enabled:
            return False, "disabled"
        if not self.audited("epilogue_vec4"):
            return False, "audit"
        if bias is not None:
            return False, "bias"
        if out_dtype != torch.bfloat16:
            return False, "out_dtype"
        if accumulator.dtype != torch.int32:
            return False, "acc_dtype"
        if row_scale.dtype != torch.float32:
            return False, "row_scale_dtype"
        if col_scale.dtype != torch.float32:
            return False, "col_scale_dtype"
        if not accumulator.is_cuda or not row_scale.is_cuda or not col_scale.is_cuda:
            return False, "device"
        if not (accumulator.device == row_scale.device == col_scale.device):
            return False, "device_mismatch"
        if not accumulator.is_contiguous():
            return False, "acc_noncontiguous"
        if not row_scale.is_contiguous():
            return False, "row_scale_noncontiguous"
        if not col_scale.is_contiguous():
            return False, "col_scale_noncontiguous"
        if accumulator.dim() != 2 or accumulator.shape[0] not in LOCAL_M:
            return False, "M"
        if accumulator.shape[1] not in EPILOGUE_N:
            return False, "N"
        if row_scale.dim() != 1 or row_scale.numel() != accumulator.shape[0]:
            return False, "row_scale_shape"
        if col_scale.dim() != 1 or col_scale.numel() != accumulator.shape[1]:
            return False, "col_scale_shape"
        if not self.is_arch(accumulator):
            return False, "arch"
        return True, "eligible"

    def unpadded_gemm_gate(self, x_8, weight_t):
        """launcher :805-818: direct GEMM only for whitelisted (M,K,N)."""
        if not self.unpadded_m_enabled:
            return False, "disabled"
        if not self.audited("int8_gemm"):
            return False, "audit"
        if not (x_8.is_cuda and weight_t.is_cuda):
            return False, "device"
        if x_8.dtype != torch.int8 or weight_t.dtype != torch.int8:
            return False, "dtype"
        if x_8.dim() != 2 or weight_t.dim() != 2 or x_8.shape[1] != weight_t.shape[0]:
            return False, "shape"
        # everything the kernel wrapper would reject is a counted refusal here, so such a
        # call reaches the host's GEMM (which accepts any layout) instead of raising
        if x_8.device != weight_t.device:
            return False, "device_mismatch"
        if not x_8.is_contiguous():
            return False, "noncontiguous"
        stride = weight_t.stride()
        if stride is not None and tuple(stride) != (1, weight_t.shape[0]):
            return False, "weight_layout"    # not the transpose view of a contiguous [N,K] weight
        if (x_8.shape[0], x_8.shape[1], weight_t.shape[1]) not in GEMM_SHAPES:
            return False, "MKN"
        if not self.is_arch(x_8):
            return False, "arch"
        return True, "eligible"

    def fused_gemm_gate(self, x_8, row_scale, weight, col_scale, bias, out_dtype):
        """GEMM with the epilogue fused: the union of the GEMM and epilogue contracts
        (bias allowed: bf16 or fp32)."""
        if not self.fused_gemm_enabled:
            return False, "disabled"
        if not self.audited("int8_gemm_dequant"):
            return False, "audit"
        if out_dtype != torch.bfloat16:
            return False, "out_dtype"
        if x_8.dtype != torch.int8 or weight.dtype != torch.int8:
            return False, "dtype"
        if row_scale.dtype != torch.float32 or col_scale.dtype != torch.float32:
            return False, "scale_dtype"
        if bias is not None and bias.dtype not in (torch.bfloat16, torch.float32):
            return False, "bias_dtype"
        if not (x_8.is_cuda and weight.is_cuda and row_scale.is_cuda and col_scale.is_cuda):
            return False, "device"
        if not (x_8.device == weight.device == row_scale.device == col_scale.device):
            return False, "device_mismatch"
        if bias is not None and not (bias.is_cuda and bias.device == x_8.device):
            return False, "bias_device"
        if not (x_8.is_contiguous() and weight.is_contiguous() and row_scale.is_contiguous()
                and col_scale.is_contiguous()):
            return False, "noncontiguous"
        if bias is not None and not bias.is_contiguous():
            return False, "bias_noncontiguous"
        if x_8.dim() != 2 or weight.dim() != 2 or x_8.shape[1] != weight.shape[1]:
            return False, "shape"
        if bias is not None and bias.numel() not in (0, weight.shape[0]):
            return False, "bias_shape"
        if (x_8.shape[0], x_8.shape[1], weight.shape[0]) not in GEMM_SHAPES:
            return False, "MKN"
        if row_scale.numel() != x_8.shape[0] or col_scale.numel() != weight.shape[0]:
            return False, "scale_shape"
        if not self.is_arch(x_8):
            return False, "arch"
        return True, "eligible"

    def weight_layout_eligible(self, weight) -> bool:
        """launcher :258-289 / :309-336 keep a (N,K) whitelist for the prepacked weight
        layout.  tcgen05 consumes the [N,K] K-major storage as is, so there is no
        prepack here; only the whitelist check on (N,K) survives."""
        return (weight.dtype == torch.int8 and weight.dim() == 2
                and tuple(weight.shape) in WEIGHT_SHAPES and weight.is_contiguous()
                and self.is_arch(weight))

    # ---- gated operator calls ----------------------------------------------------
    def quantize_activation(self, x, stochastic_rounding: int = 0):
        """launcher :182-207."""
        ok, reason = self.exact_quantizer_gate(x, stochastic_rounding)
        c = self.counters["exact_quantizer"]
        if ok:
            c.hit()
            return ops.quantize_int8_rowwise(x)
        c.refuse(reason, getattr(x, "shape", None), dtype=x.dtype, contiguous=x.is_contiguous())
        return self._fallback("quantize")(x, stochastic_rounding=stochastic_rounding)

    def swiglu_quantize_activation(self, x, stochastic_rounding: int = 0):
        ok, reason = self.swiglu_quant_gate(x, stochastic_rounding)
        c = self.counters["swiglu_quant"]
        if ok:
            c.hit()
            return ops.swiglu_quantize_int8_rowwise(x)
        c.refuse(reason, getattr(x, "shape", None), dtype=x.dtype, contiguous=x.is_contiguous())
        return self._fallback("swiglu_quantize")(x, stochastic_rounding=stochastic_rounding)

    def mod_scale_shift(self, x, scale, shift):
        ok, reason = self.mod_scale_shift_gate(x, scale, shift)
        c = self.counters["mod_scale_shift"]
        if ok:
            c.hit()
            return ops.mod_scale_shift_(x, scale, shift)
        c.refuse(reason, getattr(x, "shape", None), dtype=x.dtype)
        return self._fallback("mod_scale_shift")(x, scale, shift)

    def int8_matmul(self, x_8, weight_t):
        """launcher :805-824."""
        ok, reason = self.unpadded_gemm_gate(x_8, weight_t)
        c = self.counters["unpadded_gemm"]
        if ok:
            c.hit()
            return ops.int_mm(x_8, weight_t)
        c.refuse(reason, (x_8.shape[0], x_8.shape[1], weight_t.shape[1]))
        return self._fallback("int_mm")(x_8, weight_t)

    def dump_counters(self) -> dict:
        out = {k: v.summary() for k, v in self.counters.items()}
        out["flash"]["head_chunk_calls"] = self.flash_head_chunk_calls
        return out

    def log_counters(self) -> None:
        log.warning("B200 gate counters %s", json.dumps(self.dump_counters(), sort_keys=True))


def agree_flag_across_ranks(flag: bool, group=None) -> None:
    """Every rank must run with the same head-chunk-overlap setting (launcher
    :1281-1297): all-gather one int32 per rank and raise on disagreement."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return
    backend = dist.get_backend(group)
    device = (torch.device("cuda", torch.cuda.current_device()) if backend == "nccl"
              else torch.device("cpu"))
    local = torch.tensor([int(flag)], device=device, dtype=torch.int32)
    gathered = [torch.empty_like(local) for _ in range(dist.get_world_size(group))]
    dist.all_gather(gathered, local, group=group)
    if any(int(g.item()) != int(local.item()) for g in gathered):
        raise RuntimeError("head-chunk overlap flag differs between distributed ranks")


_default: Gates | None = None


def default_gates() -> Gates:
    """Process-wide gate configuration built from the environment on first use; its
    counters are logged at exit like the reference's (launcher :210-222)."""
    global _default
    if _default is None:
        _default = Gates.from_env()
        atexit.register(_default.log_counters)
    return _default
