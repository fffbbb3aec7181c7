"""Gated attention entry point.

Mirror of `_h3_flash_attention` in the reference
(launcher/benchmark_launcher_v14_hires_int8_candidate.py:1152-1276): the flash
kernel is used only when the complete contract matches; otherwise the call is
counted, its signature logged (at most 8 distinct ones) and forwarded to the host's
original attention with the original arguments.  Generalised from the reference's
single deployment (28 heads, 2 ranks, gfx936) to heads in {24,12,6,3} (= 24 / SP
degree) and SP degrees 1/2/4/8, keeping both admitted stride families:
  standard layout     q/k/v are [S,h,128] storage viewed as [1,h,S,128]:
                      stride()[1:] == (128, h*128, 1)
  head-chunk layout   views into a packed [S,c,3,128] all-to-all receive buffer:
                      stride()[1:] == (384, c*384, 1)   (overlap flag required)
plus the packed qkv projection output [S,3,h,128] viewed per part:
                      stride()[1:] == (128, 3*h*128, 1)
"""
from __future__ import annotations

import logging

import torch

from . import ops
from .gates import (FLASH_HEADS, FLASH_HEAD_CHUNKS, FLASH_MAX_SEQ, SP_WORLDS, Gates,
                    default_gates)

log = logging.getLogger("b2dit.attention")


class SPContext:
    """What the gate needs to know about sequence parallelism (the reference reads
    these fields from its host's `attention_context`, launcher :1169-1173)."""

    def __init__(self, rank: int = 0, world_size: int = 1, sequence_splits=None,
                 local_length: int | None = None):
        self.rank = rank
        self.world_size = world_size
        self.sequence_splits = tuple(sequence_splits) if sequence_splits is not None else None
        self.local_length = local_length


# key of the host's `transformer_options` dict under which the sequence-parallel state
# travels (an SPContext-like object or a dict with the same four fields)
SP_OPTIONS_KEY = "sequence_parallel"


def context_from_transformer_options(transformer_options):
    """Default context resolver: what the reference obtains from its host with
    `attention_context(kwargs["transformer_options"])` (launcher :1167-1173).

    Not a dict -> None (the call is refused with `sp_world`, as in the reference).  A dict
    without sequence-parallel state describes a single-GPU run: world size 1.  Otherwise the
    entry under SP_OPTIONS_KEY is used: any object with `world_size` (and optionally `rank`,
    `sequence_splits`, `local_length`), or a dict with those keys.  A host whose model keeps
    this state elsewhere registers its own resolver on the Gates object."""
    if not isinstance(transformer_options, dict):
        return None
    state = transformer_options.get(SP_OPTIONS_KEY)
    if state is None:
        return SPContext(0, 1)
    if isinstance(state, dict):
        return SPContext(state.get("rank", 0), state.get("world_size", 1),
                         state.get("sequence_splits"), state.get("local_length"))
    return state if hasattr(state, "world_size") else None


def resolve_precision(attn_precision, dtype):
    """Default precision resolver: the requested precision as given.  A host that can force
    an fp32 upcast regardless of the argument (the reference calls its host's
    `get_attn_precision(attn_precision, query.dtype)`, launcher :1165) registers that
    function on the Gates object, so a forced upcast is refused with `precision`."""
    return attn_precision


def expected_splits(seq: int, world: int) -> tuple[int, ...]:
    base, rem = divmod(seq, world)
    return tuple(base + (1 if r < rem else 0) for r in range(world))


def flash_gate(g: Gates, query, key, value, heads, mask, skip_reshape, kwargs, sp_context,
               resolved_precision=None):
    """(eligible, reason, is_head_chunk_layout); conditions of launcher :1174-1209."""
    if not g.flash_enabled:
        return False, "disabled", False
    if not g.audited("flash_fwd"):
        return False, "audit", False
    tensors = (query, key, value)
    if mask is not None:
        return False, "mask", False
    if not skip_reshape:
        return False, "skip_reshape", False
    if "scale" in kwargs:
        return False, "scale", False
    if kwargs.get("enable_gqa", False):
        return False, "gqa", False
    if resolved_precision == torch.float32:
        return False, "precision", False
    if sp_context is None or sp_context.world_size not in SP_WORLDS:
        return False, "sp_world", False
    if query.dtype != torch.bfloat16 or any(t.dtype != query.dtype for t in tensors):
        return False, "dtype", False
    if query.device.type != "cuda" or any(t.device != query.device for t in tensors):
        return False, "device", False
    if not (query.shape == key.shape == value.shape):
        return False, "shape_mismatch", False
    if any(t.requires_grad for t in tensors):
        return False, "requires_grad", False
    if query.ndim != 4 or query.shape[0] != 1 or query.shape[3] != 128:
        return False, "layout", False
    if not (1 <= query.shape[2] <= FLASH_MAX_SEQ):
        return False, "sequence", False
    h = query.shape[1]
    standard = (heads == h and h in FLASH_HEADS and all(
        tuple(t.stride()[1:]) in ((128, h * 128, 1), (128, 3 * h * 128, 1)) for t in tensors))
    head_chunk = (
        g.head_chunk_overlap_enabled and heads == h and h in FLASH_HEAD_CHUNKS
        and all(tuple(t.stride()[1:]) == (384, h * 384, 1) for t in tensors)
        and sp_context.sequence_splits is not None
        and sp_context.sequence_splits == expected_splits(query.shape[2], sp_context.world_size)
        and sp_context.local_length == sp_context.sequence_splits[sp_context.rank])
    if not (standard or head_chunk):
        return False, "layout", False
    if not g.is_arch(query):
        return False, "arch", False
    return True, "eligible", head_chunk and not standard


def attention(query, key, value, heads, mask=None, attn_precision=None, skip_reshape=False,
              skip_output_reshape=False, gates: Gates | None = None, sp_context=None, **kwargs):
    """Drop-in for the host's `optimized_attention(q, k, v, heads, ...)`.

    The sequence-parallel context comes from `kwargs["transformer_options"]` through the
    gates' `context_resolver` (what the reference does, launcher :1167-1173) unless the caller
    passes `sp_context=` explicitly; the precision the gate tests and logs is the one the
    gates' `precision_resolver` returns for (attn_precision, query.dtype) (launcher :1165)."""
    g = gates if gates is not None else default_gates()
    if sp_context is None:
        resolver = getattr(g, "context_resolver", None) or context_from_transformer_options
        sp_context = resolver(kwargs.get("transformer_options"))
    precision = (getattr(g, "precision_resolver", None) or resolve_precision)(attn_precision, query.dtype)
    ok, reason, chunked = flash_gate(g, query, key, value, heads, mask, skip_reshape, kwargs,
                                     sp_context, precision)
    c = g.counters["flash"]
    if not ok:
        tensors = (query, key, value)
        signature = (tuple(query.shape), tuple(tuple(t.stride()) for t in tensors), heads,
                     mask is not None, skip_reshape, "scale" in kwargs, str(precision),
                     getattr(sp_context, "world_size", None),
                     tuple(t.requires_grad for t in tensors))
        c.fallbacks[reason] += 1
        if signature not in g.flash_fallback_signatures and len(g.flash_fallback_signatures) < 8:
            g.flash_fallback_signatures.add(signature)
            log.warning("B200 FlashAttention FALLBACK reason=%s shape=%s strides=%s heads=%s "
                        "mask=%s skip_reshape=%s scale_present=%s precision=%s sp_rank=%s "
                        "sp_world=%s requires_grad=%s", reason, *signature[:7],
                        getattr(sp_context, "rank", None), signature[7], signature[8])
        return g._fallback("attention")(query, key, value, heads, mask=mask,
                                        attn_precision=attn_precision, skip_reshape=skip_reshape,
                                        skip_output_reshape=skip_output_reshape, **kwargs)
    c.hits += 1
    if chunked:
        g.flash_head_chunk_calls += 1
    output = ops.fwd_bhsd(query, key, value, float(query.shape[-1] ** -0.5))
    if g._flash_first_call:
        # surface an incompatible launch at the feature boundary (launcher :1262-1265)
        torch.cuda.synchronize(query.device)
        ops.check_device_status(query.device)
        log.warning("B200 FlashAttention ENABLED rank=%s shape=%s stride=%s call=%s",
                    getattr(sp_context, "rank", None), tuple(query.shape), tuple(query.stride()),
                    c.hits)
        g._flash_first_call = False
    if skip_output_reshape:
        return output
    return output.transpose(1, 2).flatten(start_dim=2)
