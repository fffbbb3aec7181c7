"""B200-native (sm_100a) drop-in for the exactness-gated DiT hot path of
dcu-video-dit-turbo: rowwise INT8 quantizer, tcgen05 INT8 GEMM with the dequant
epilogue fused, mod-scale-shift, swiglu-quant, bf16 FlashAttention forward, the
launcher's gate layer (whitelists, audit hash, counted refusal) and Ulysses
sequence parallelism around attention.

Every operator is a hand-written CUDA kernel behind the C ABI in include/b2dit.h
(libb2dit.so, built in-tree by build.py).  There is no CPU or eager fallback in
this package: importing an operator without the built library raises.

The directory name contains a hyphen, so import it with importlib
(`importlib.import_module("dcu-video-dit-turbo_b200")`); the package also
registers itself under the alias `dcu_video_dit_turbo_b200`.
"""
import sys as _sys

_sys.modules.setdefault("dcu_video_dit_turbo_b200", _sys.modules[__name__])

from . import _lib, ops, gates, linear, attention, peer, ulysses, block, dispatch, save, vae_sp  # noqa: E402,F401

__all__ = ["_lib", "ops", "gates", "linear", "attention", "peer", "ulysses", "block", "dispatch", "save", "vae_sp"]
