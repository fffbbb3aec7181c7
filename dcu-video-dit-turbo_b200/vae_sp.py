"""Temporal-chunk parallel VAE decode: the orchestration around the host's decoder.

Mirror of the reference launcher's H3_VAE_SP hook
(launcher/benchmark_launcher_v14_hires_int8_candidate.py:449-587 in the reference).  The video
VAE decodes a latent clip in temporal chunks; each chunk yields `main` frames and `overlap`
frames, consecutive chunks are cross-faded over the overlap and written one after the other.
The chunks are independent until the cross-fade, so the ranks of a sequence-parallel job
split them: rank 0 decodes and assembles the first range, every other rank decodes its range
and sends `cat(main, overlap)` packets to rank 0, which blends and appends them in order.

The decoder and the blend are the HOST APPLICATION's (its VAE is not part of the reference
tree); they are passed in as callables, and nothing here changes a value: the assembled clip
is bitwise the single-rank one (checked packet by packet in `validate` mode, as the
reference's H3_VALIDATE_VAE_SP does).  Generalised from the reference's fixed 2 ranks /
21 chunks / 17+5 frames to any world size and per-chunk frame counts (sent as a small header).
Works on NCCL (CUDA tensors) and gloo (CPU tensors; used by the tests).
"""
from __future__ import annotations

import logging
import time
from typing import Callable, Sequence

import torch
import torch.distributed as dist

log = logging.getLogger("dcu_video_dit_turbo_b200.vae_sp")


def chunk_ranges(num_chunks: int, world: int) -> list[range]:
    """Contiguous chunk ranges per rank, the first `num_chunks % world` ranks one longer
    (21 chunks on 2 ranks: 0-10 and 11-20, the reference's cut at 11)."""
    base, rem = divmod(num_chunks, world)
    out, start = [], 0
    for r in range(world):
        n = base + (1 if r < rem else 0)
        out.append(range(start, start + n))
        start += n
    return out


class TemporalChunkDecode:
    def __init__(self, num_chunks: int, output_frames: int, frame_overlap: int, group=None,
                 validate: bool = False):
        self.num_chunks = int(num_chunks)
        self.output_frames = int(output_frames)
        self.frame_overlap = int(frame_overlap)
        self.group = group
        self.validate = bool(validate)

    # -- assembly on the collecting rank ------------------------------------------------
    class _Writer:
        def __init__(self, output_frames: int):
            self.frames, self.pos, self.dec = output_frames, 0, None

        def write(self, part: torch.Tensor) -> None:
            n = part.shape[2]
            if n <= 0:
                return
            if self.dec is None:
                shape = list(part.shape)
                shape[2] = self.frames
                self.dec = torch.empty(shape, device=part.device, dtype=part.dtype)
            take = min(n, max(0, self.frames - self.pos))
            if take:
                self.dec[:, :, self.pos:self.pos + take].copy_(part[:, :, :take])
                self.pos += take

    def _assemble(self, writer, previous_overlap, main, overlap, blend):
        if previous_overlap is not None:
            main = blend(previous_overlap, main, self.frame_overlap)
        writer.write(main)
        return overlap

    def decode_single(self, z, decode_parts: Callable, blend: Callable) -> torch.Tensor:
        """The sequential decode every rank would do alone (the fallback and the oracle)."""
        writer, prev = self._Writer(self.output_frames), None
        for index in range(self.num_chunks):
            main, overlap = decode_parts(z, index)
            prev = self._assemble(writer, prev, main, overlap, blend)
        writer.write(prev)
        if writer.pos != self.output_frames:
            raise RuntimeError(f"assembled {writer.pos} frames, expected {self.output_frames}")
        return writer.dec

    # -- the parallel decode --------------------------------------------------------------
    def decode(self, z: torch.Tensor, decode_parts: Callable, blend: Callable):
        """`decode_parts(z, index) -> (main, overlap)` frames on dim 2; `blend(previous_overlap,
        main, frame_overlap) -> main`.  Returns the assembled clip on rank 0 and None on the
        other ranks (they have nothing to save)."""
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(self.group) == 1:
            return self.decode_single(z, decode_parts, blend)
        rank, world = dist.get_rank(self.group), dist.get_world_size(self.group)
        z = z.contiguous()
        dist.broadcast(z, src=0, group=self.group)          # every rank decodes the same latents
        ranges = chunk_ranges(self.num_chunks, world)
        started = time.perf_counter()
        if rank != 0:
            parts = [decode_parts(z, index) for index in ranges[rank]]
            header = torch.tensor([[m.shape[2], o.shape[2]] for m, o in parts] or [[0, 0]],
                                  dtype=torch.int64, device=z.device)
            local = time.perf_counter() - started
            if len(ranges[rank]):
                dist.send(header, dst=0, group=self.group)
                for main, overlap in parts:
                    dist.send(torch.cat((main, overlap), dim=2).contiguous(), dst=0, group=self.group)
            log.warning("B200_VAE_SP_TIMING rank=%d chunks=%d local_seconds=%.6f", rank,
                        len(ranges[rank]), local)
            return None

        writer, prev = self._Writer(self.output_frames), None
        for index in ranges[0]:
            main, overlap = decode_parts(z, index)
            prev = self._assemble(writer, prev, main, overlap, blend)
        local = time.perf_counter() - started
        if prev is None:
            raise RuntimeError("rank 0 needs at least one chunk")
        received_started = time.perf_counter()
        for src in range(1, world):
            if not len(ranges[src]):
                continue
            header = torch.empty((len(ranges[src]), 2), dtype=torch.int64, device=z.device)
            dist.recv(header, src=src, group=self.group)
            for index, (n_main, n_overlap) in zip(ranges[src], header.tolist()):
                shape = list(prev.shape)
                shape[2] = n_main + n_overlap
                packet = torch.empty(shape, device=z.device, dtype=prev.dtype)
                dist.recv(packet, src=src, group=self.group)
                if self.validate:
                    want = torch.cat(decode_parts(z, index), dim=2)
                    if not torch.equal(want, packet):
                        err = (want.float() - packet.float()).abs().max().item()
                        raise RuntimeError(f"rank {src} VAE chunk {index} is not bitwise exact; max_abs={err}")
                prev = self._assemble(writer, prev, packet[:, :, :n_main], packet[:, :, n_main:], blend)
        writer.write(prev)
        if writer.pos != self.output_frames:
            raise RuntimeError(f"assembled {writer.pos} frames, expected {self.output_frames}")
        log.warning("B200_VAE_SP_TIMING rank=0 chunks=%d local_seconds=%.6f receive_seconds=%.6f validate=%s",
                    len(ranges[0]), local, time.perf_counter() - received_started, self.validate)
        return writer.dec
