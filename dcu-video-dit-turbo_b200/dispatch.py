"""Launcher-level integration: how a model's ordinary `linear` calls reach the INT8 path.

Three pieces of the reference launcher
(launcher/benchmark_launcher_v14_hires_int8_candidate.py in the reference):

  * :292-343  a layout handler registered for `aten.linear` on the host application's
    quantized-tensor class: an eligible call (plain activation, un-transposed int8 weight
    with a whitelisted [N,K] shape on the right architecture) goes to the INT8 linear,
    anything else to the original handler.  Here `Int8Weight` is that tensor class (the
    host's class is not part of the reference tree): a wrapper subclass whose
    `torch.nn.functional.linear` is dispatched by `LinearDispatch`.
    The reference also re-stores the weight column-major for its GEMM library (:258-289);
    tcgen05 reads the [N,K] K-major storage as it is, so no prepack exists here.
  * :1068-1094  SIGUSR1 / SIGUSR2 switch the INT8 route on and off in a running process.
  * launcher/coordinator.py:110-122  every rank of a sequence-parallel job is handed the
    sha256 of the canonical JSON of (prompt, conditioning hashes); `job_digest` computes
    it and `agree_digest_across_ranks` refuses to run when ranks disagree.

All of this is host code; the kernels are reached through `linear.int8_linear`.
"""
from __future__ import annotations

import hashlib
import json
import logging
import signal
from typing import Callable

import torch

from . import linear as _linear
from .gates import Gates, default_gates

log = logging.getLogger("dcu_video_dit_turbo_b200.dispatch")


class Int8Weight(torch.Tensor):
    """Per-output-channel (or per-tensor) symmetric INT8 weight that behaves as a bf16
    [N,K] tensor: `qdata` int8 [N,K], `scale` fp32 [N] or scalar, weight = qdata * scale."""

    @staticmethod
    def __new__(cls, qdata: torch.Tensor, scale: torch.Tensor, transposed: bool = False,
                dispatch: "LinearDispatch | None" = None):
        if qdata.dtype != torch.int8 or qdata.dim() != 2:
            raise ValueError("qdata must be int8 [N,K]")
        shape = tuple(reversed(qdata.shape)) if transposed else tuple(qdata.shape)
        return torch.Tensor._make_wrapper_subclass(cls, shape, dtype=torch.bfloat16,
                                                   device=qdata.device, requires_grad=False)

    def __init__(self, qdata, scale, transposed=False, dispatch=None):
        self.qdata = qdata
        self.scale = scale.to(torch.float32)
        self.transposed = bool(transposed)
        self.dispatch = dispatch

    def get_plain_tensors(self):
        return self.qdata, self.scale

    def dequantize(self) -> torch.Tensor:
        w = (self.qdata.float() * self.scale.reshape(-1, 1).to(self.qdata.device)).to(torch.bfloat16)
        return w.t() if self.transposed else w

    def __repr__(self):  # the default repr would try to read wrapper storage
        return (f"Int8Weight(shape={tuple(self.shape)}, device={self.device}, "
                f"transposed={self.transposed})")

    @classmethod
    def __torch_function__(cls, func, types, args=(), kwargs=None):
        kwargs = kwargs or {}
        if func is torch.nn.functional.linear:
            weight = args[1] if len(args) > 1 else kwargs.get("weight")
            if isinstance(weight, Int8Weight):
                d = weight.dispatch if weight.dispatch is not None else default_dispatch()
                return d.linear(*args, **kwargs)
        with torch._C.DisableTorchFunctionSubclass():
            return func(*args, **kwargs)

    @classmethod
    def __torch_dispatch__(cls, func, types, args=(), kwargs=None):
        raise NotImplementedError(
            f"{func} on an Int8Weight: only torch.nn.functional.linear is dispatched; call "
            f".dequantize() for anything else")


class LinearDispatch:
    """Routes `linear(input, Int8Weight, bias)`; counts what it routed where."""

    def __init__(self, gates: Gates | None = None, enabled: bool = True):
        self.gates = gates
        self.enabled = bool(enabled)
        self.routed = 0
        self.fallbacks: dict[str, int] = {}
        self._original: Callable | None = None

    # -- the handler ----------------------------------------------------------------
    def register_original_handler(self, fn: Callable) -> None:
        """`fn(input, weight: Int8Weight, bias)`: the host's own handler, called (and
        counted) for calls this dispatch refuses.  Without one a refused call raises, like
        every gate of this package: nothing here computes on a silent substitute path.
        `dequantized_linear` is a ready-made handler."""
        self._original = fn

    def _refuse(self, reason: str, inp, weight, bias):
        n = self.fallbacks.get(reason, 0) + 1
        self.fallbacks[reason] = n
        if n == 1 or n % 1000 == 0:
            log.warning("INT8 linear dispatch fallback reason=%s count=%d weight=%s", reason, n,
                        tuple(weight.shape))
        if self._original is None:
            raise RuntimeError(f"INT8 linear dispatch refused the call ({reason}) and no original "
                               f"handler is registered")
        return self._original(inp, weight, bias)

    def eligibility(self, inp, weight: Int8Weight) -> str:
        """'eligible' or the first failing condition, in the reference handler's order."""
        g = self.gates if self.gates is not None else default_gates()
        if not self.enabled:
            return "disabled"
        if weight.transposed:
            return "transposed"
        if isinstance(inp, Int8Weight):
            return "quantized_input"
        if not g.weight_layout_eligible(weight.qdata):
            return "weight_shape_or_arch"
        return "eligible"

    def linear(self, inp, weight: Int8Weight, bias=None, out_dtype: torch.dtype | None = None):
        reason = self.eligibility(inp, weight)
        if reason != "eligible":
            return self._refuse(reason, inp, weight, bias)
        g = self.gates if self.gates is not None else default_gates()
        self.routed += 1
        qdata, scale = weight.get_plain_tensors()
        return _linear.int8_linear(inp.contiguous(), qdata, scale, bias,
                                   out_dtype=out_dtype or inp.dtype, gates=g)

    # -- run-time toggles (launcher :1068-1094) ----------------------------------------
    def set_enabled(self, enabled: bool) -> None:
        self.enabled = bool(enabled)
        log.warning("B200 INT8 linear path %s", "ENABLED" if self.enabled else "DISABLED")

    def install_signal_toggles(self, on=signal.SIGUSR1, off=signal.SIGUSR2):
        """SIGUSR1 enables, SIGUSR2 disables; returns the previous handlers."""
        prev_on = signal.signal(on, lambda _s, _f: self.set_enabled(True))
        prev_off = signal.signal(off, lambda _s, _f: self.set_enabled(False))
        return prev_on, prev_off

    def summary(self) -> dict:
        return {"enabled": self.enabled, "routed": self.routed, "fallbacks": dict(self.fallbacks)}


def dequantized_linear(inp, weight: Int8Weight, bias=None):
    """Original-handler stand-in for hosts without one: dequantize the weight, bf16 linear."""
    x = inp.dequantize() if isinstance(inp, Int8Weight) else inp
    b = None if bias is None else bias.to(x.dtype)
    return torch.nn.functional.linear(x, weight.dequantize().to(x.dtype), b)


_default: LinearDispatch | None = None


def default_dispatch() -> LinearDispatch:
    global _default
    if _default is None:
        _default = LinearDispatch()
    return _default


def quantize_weight(weight: torch.Tensor, dispatch: LinearDispatch | None = None) -> Int8Weight:
    """bf16/fp32 [N,K] -> Int8Weight with per-output-channel symmetric scales
    (scale = absmax/127, round half even, clamp to +-127), as the benchmark's weights are
    prepared."""
    w = weight.float()
    absmax = w.abs().amax(dim=1)
    # tensor / tensor is an IEEE division on every device (a Python-scalar divisor is turned
    # into a multiplication by its reciprocal on CUDA, which changes the last bit)
    scale = (absmax / torch.full_like(absmax, 127.0)).clamp(min=1e-30)
    q = torch.clamp(torch.round(w / scale.reshape(-1, 1)), -127, 127).to(torch.int8)
    return Int8Weight(q.contiguous(), scale, dispatch=dispatch)


# -- job digest (launcher/coordinator.py:110-122) -------------------------------------------
def job_digest(prompt: dict, conditioning_inputs: dict | None = None, **extra) -> str:
    """sha256 of the canonical JSON (sorted keys, compact separators, UTF-8) of the job
    contract.  `extra` (seed, gate flags, ...) is included only when given, so the bare
    two-field form equals the reference coordinator's digest for the same prompt."""
    contract = {"prompt": prompt, "conditioning_inputs": conditioning_inputs or {}}
    contract.update(extra)
    canonical = json.dumps(contract, ensure_ascii=False, sort_keys=True,
                           separators=(",", ":")).encode("utf-8")
    return hashlib.sha256(canonical).hexdigest()


def agree_digest_across_ranks(digest: str, group=None) -> None:
    """Raises on every rank when the ranks of a sequence-parallel job hold different job
    digests (different prompt, seed or flags would otherwise produce silent garbage)."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()):
        return
    raw = bytes.fromhex(digest)
    if len(raw) != 32:
        raise ValueError("digest must be a sha256 hex string")
    backend = dist.get_backend(group)
    device = (torch.device("cuda", torch.cuda.current_device()) if backend == "nccl"
              else torch.device("cpu"))
    local = torch.tensor(list(raw), dtype=torch.uint8, device=device)
    gathered = [torch.empty_like(local) for _ in range(dist.get_world_size(group))]
    dist.all_gather(gathered, local, group=group)
    if any(not torch.equal(g, local) for g in gathered):
        raise RuntimeError("job digest differs between distributed ranks")
