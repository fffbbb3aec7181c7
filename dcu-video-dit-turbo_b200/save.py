"""Batched 8-bit frame conversion for the video writer.

Mirror of the reference launcher's H3_SAVE_BATCH_U8 hook
(launcher/benchmark_launcher_v14_hires_int8_candidate.py:607-723 in the reference): the host
application's writer converts and copies one frame at a time (three tiny launches and a
synchronous device-to-host copy per frame); an eligible clip is instead converted by ONE
kernel and fetched by ONE copy, and the same RGB24 frames go to the same encoder.  Encoding,
muxing and audio stay with the host application (they are not GPU work); a refused clip goes
to the writer the host registers, or raises.
"""
from __future__ import annotations

import logging
import os
import time
from typing import Callable

import torch

from . import ops

log = logging.getLogger("dcu_video_dit_turbo_b200.save")


class BatchU8Save:
    def __init__(self, enabled: bool | None = None):
        self.enabled = (os.environ.get("H3_SAVE_BATCH_U8", "0") == "1") if enabled is None else bool(enabled)
        self.hits = 0
        self.fallbacks: dict[str, int] = {}
        self._original: Callable | None = None

    def register_original_writer(self, fn: Callable) -> None:
        """`fn(images, bit_depth)` -> frames, the host's per-frame path, for refused clips."""
        self._original = fn

    def gate(self, images, bit_depth: int) -> tuple[bool, str]:
        """Eligibility in the reference hook's order (:625-630), with `disabled` and `device`
        in front: 8-bit output, a [frames, height, width, 3] tensor."""
        if not self.enabled:
            return False, "disabled"
        if bit_depth >= 10:
            return False, "bit_depth"
        if not isinstance(images, torch.Tensor):
            return False, "not_tensor"
        if images.ndim != 4:
            return False, "rank"
        if images.shape[-1] != 3:
            return False, "channels"
        if not images.is_cuda:
            return False, "device"
        if images.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            return False, "dtype"
        return True, "eligible"

    def frames_u8(self, images, bit_depth: int = 8) -> torch.Tensor:
        """uint8 [frames, height, width, 3] in (pinned) host memory, ready for the encoder."""
        ok, reason = self.gate(images, bit_depth)
        if not ok:
            self.fallbacks[reason] = self.fallbacks.get(reason, 0) + 1
            if self._original is None:
                raise RuntimeError(f"batched 8-bit save refused the clip ({reason}) and no original "
                                   f"writer is registered")
            return self._original(images, bit_depth)
        started = time.perf_counter()
        device_u8 = ops.images_to_u8(images.contiguous())      # contiguous() changes layout only
        host = torch.empty(device_u8.shape, dtype=torch.uint8, pin_memory=True)
        host.copy_(device_u8, non_blocking=True)
        torch.cuda.current_stream(images.device).synchronize()
        self.hits += 1
        log.warning("B200_BATCH_SAVE_TIMING quantize_d2h_seconds=%.6f frames=%d",
                    time.perf_counter() - started, images.shape[0])
        return host
