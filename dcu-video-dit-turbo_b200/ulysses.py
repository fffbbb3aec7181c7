"""Ulysses sequence parallelism around attention, over torch.distributed.

Tokens are sharded across ranks (uneven splits allowed: the first S mod P ranks
hold one extra row); attention needs every token, so an all-to-all turns the
token-sharded [L_r, H, D] tensors into head-sharded [S, H/P, D] ones, attention
runs on the local heads, and a second all-to-all goes back.  Byte layouts follow
the reference's in-tree model of its sequence-parallel code
(benchmarks/bench_sp_head_chunk_overlap.py:83-193 in the reference):
  sequence_to_heads / heads_to_sequence   :83-118
  packed QKV head chunk [world, L, c, 3, D] -> [S, c, 3, D]   :140-164
  chunk i attention overlapped with chunk i+1's all-to-all on a side stream   :179-193
generalised from 2 ranks to any world size dividing the head count.

Works on the NCCL backend (CUDA tensors, NVLink) and on gloo (CPU tensors; used
by the layout tests).  Received data always lands in local memory before a kernel
reads it.  Two transports carry the same layouts: all-to-all collectives
(`attention_packed`), and, for the ranks of one machine, the kernels' own stores into the
destination rank's memory (`enable_peer_exchange` + `attention_peer`; peer.py), which
removes both all-to-alls and their pack / unpack passes from the step.
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch
import torch.distributed as dist

from .peer import PeerExchange


def sequence_splits(seq: int, world: int) -> tuple[int, ...]:
    base, rem = divmod(seq, world)
    return tuple(base + (1 if r < rem else 0) for r in range(world))


def choose_head_chunks(seq: int, local_heads: int, sms: int = 148, q_rows_per_cta: int = 256,
                       target: float = 0.9, max_chunks: int = 4) -> int:
    """How many head chunks to split a rank's attention into.

    More chunks hide more of the all-to-all behind attention, but every chunk is its own
    attention launch of ceil(seq / q_rows_per_cta) * heads_per_chunk CTAs on `sms` SMs, and a
    launch that fills a fraction of a wave leaves SMs idle (93 CTAs on 148 SMs at 23638
    tokens and one head per chunk).  Picks the largest divisor of `local_heads` whose
    launches keep at least `target` of their last wave busy, else the most efficient one;
    never more than `max_chunks` (the exposed share of the transfer is 1/chunks already)."""
    ctas_per_head = -(-seq // q_rows_per_cta)
    best, best_eff = 1, 0.0
    for chunks in range(min(local_heads, max_chunks), 0, -1):
        if local_heads % chunks:
            continue
        waves = ctas_per_head * (local_heads // chunks) / sms
        eff = waves / -(-waves // 1)
        if eff >= target:
            return chunks
        if eff > best_eff:
            best, best_eff = chunks, eff
    return best


class UlyssesSP:
    def __init__(self, splits: Sequence[int], heads: int, dim: int = 128, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if len(splits) != self.world:
            raise RuntimeError(f"need {self.world} sequence splits, got {len(splits)}")
        if heads % self.world:
            raise RuntimeError("world size must divide the head count")
        self.splits = tuple(int(s) for s in splits)
        self.local_length = self.splits[self.rank]
        self.sequence = sum(self.splits)
        self.heads = heads
        self.local_heads = heads // self.world
        self.dim = dim
        self.row0 = sum(self.splits[:self.rank])
        self._comm_stream = None
        self.peer: PeerExchange | None = None

    # -- exchange through peer memory ---------------------------------------------------
    def enable_peer_exchange(self, device: torch.device) -> PeerExchange:
        """Allocate and map the peer buffers of this group (collective; all ranks on one
        machine with peer access between their GPUs).  Raises RuntimeError when a buffer
        cannot be allocated or mapped; the all-to-all path stays usable then."""
        if self.peer is None:
            self.peer = PeerExchange(self.splits, self.heads, self.dim, device, self.group)
        return self.peer

    def attention_peer(self, scatter: Callable, attn: Callable) -> torch.Tensor:
        """Sequence-parallel attention without all-to-all collectives.

        `scatter(recv_table, row0, sequence)` must launch ops.qk_norm_rope_scatter for this
        rank's rows (it stores q, k, v of every head into the owner rank's receive buffer).
        Then: rank barrier, attention over the H/P local heads on the local receive buffer,
        one copy kernel that pushes every owner's rows of the output into its gathered buffer,
        rank barrier.  Returns the gathered buffer [1, P, L_r, H/P, D] (same layout as
        `attention_packed` with one chunk), which is REUSED by the next call.

        Everything runs on the current stream, and a step's calls must be issued on the same
        stream on every rank: the second barrier of step t orders every rank's attention
        reads before any rank's scatter of step t+1, and the first barrier of step t+1 orders
        every rank's reads of the gathered buffer before any push of step t+1."""
        pe = self.peer
        if pe is None:
            raise RuntimeError("enable_peer_exchange() has not been called on this group")
        scatter(pe.recv_buffer.table, self.row0, self.sequence)
        pe.barrier()
        out = attn(*self.chunk_views(pe.recv[0]))                  # [1,c,S,D] view of [1,S,c,D]
        rows = out.transpose(1, 2).reshape(self.sequence, self.local_heads, self.dim)
        pe.push(rows)
        pe.barrier()
        return pe.result

    # -- plain transforms ----------------------------------------------------------
    def sequence_to_heads(self, tensor: torch.Tensor) -> torch.Tensor:
        """[L_r, H, D] -> [S, H/P, D]."""
        L, hl, d = self.local_length, self.local_heads, self.dim
        send = tensor.reshape(L, self.world, hl, d).permute(1, 0, 2, 3).contiguous().reshape(-1)
        recv = torch.empty(self.sequence * hl * d, device=tensor.device, dtype=tensor.dtype)
        dist.all_to_all_single(recv, send,
                               output_split_sizes=[s * hl * d for s in self.splits],
                               input_split_sizes=[L * hl * d] * self.world, group=self.group)
        return recv.view(self.sequence, hl, d)

    def heads_to_sequence(self, tensor: torch.Tensor) -> torch.Tensor:
        """[S, H/P, D] -> [L_r, H, D]."""
        L, hl, d = self.local_length, self.local_heads, self.dim
        send = tensor.contiguous().reshape(-1)  # rows are already grouped by owner rank
        recv = torch.empty(self.world * L * hl * d, device=tensor.device, dtype=tensor.dtype)
        dist.all_to_all_single(recv, send,
                               output_split_sizes=[L * hl * d] * self.world,
                               input_split_sizes=[s * hl * d for s in self.splits],
                               group=self.group)
        return recv.view(self.world, L, hl, d).permute(1, 0, 2, 3).reshape(L, self.heads, d)

    # -- packed QKV head chunks ------------------------------------------------------
    def pack_chunk(self, qkv: torch.Tensor, start: int, stop: int, async_op: bool):
        """qkv is the packed projection output [L_r, 3, H, D].  Sends heads
        [start, stop) of every rank's head group as [world, L_r, c, 3, D] and receives
        [S, c, 3, D].  Returns (receive, send, work)."""
        L, hl, d = self.local_length, self.local_heads, self.dim
        c = stop - start
        src = qkv.view(L, 3, self.world, hl, d)[:, :, :, start:stop]      # [L,3,P,c,D]
        send = torch.empty((self.world, L, c, 3, d), device=qkv.device, dtype=qkv.dtype)
        send.copy_(src.permute(2, 0, 3, 1, 4))
        recv = torch.empty((self.sequence, c, 3, d), device=qkv.device, dtype=qkv.dtype)
        work = dist.all_to_all_single(recv.reshape(-1), send.reshape(-1),
                                      output_split_sizes=[s * c * 3 * d for s in self.splits],
                                      input_split_sizes=[L * c * 3 * d] * self.world,
                                      group=self.group, async_op=async_op)
        return recv, send, work

    @staticmethod
    def chunk_views(recv: torch.Tensor):
        """[S, c, 3, D] -> q, k, v as [1, c, S, D] views with strides (., 384, c*384, 1)."""
        q, k, v = recv.unbind(dim=2)
        return tuple(t.transpose(0, 1).unsqueeze(0) for t in (q, k, v))

    # -- pre-packed exchange (no pack / unpack copies) ------------------------------------
    def exchange_packed(self, send: torch.Tensor, async_op: bool = False):
        """One chunk's all-to-all: send [world, L_r, c, 3, D] (already destination-major)
        -> receive [S, c, 3, D].  Returns (receive, work)."""
        _, L, c, three, d = send.shape
        recv = torch.empty((self.sequence, c, three, d), device=send.device, dtype=send.dtype)
        work = dist.all_to_all_single(recv.reshape(-1), send.reshape(-1),
                                      output_split_sizes=[s * c * three * d for s in self.splits],
                                      input_split_sizes=[L * c * three * d] * self.world,
                                      group=self.group, async_op=async_op)
        return recv, work

    def reverse_into(self, out_chunk: torch.Tensor, recv_slot: torch.Tensor, async_op: bool = False):
        """Reverse all-to-all of one chunk's attention output [S, c, D] (contiguous; rows are
        already grouped by owner rank) into recv_slot [world, L_r, c, D]."""
        c, d = out_chunk.shape[1], out_chunk.shape[2]
        L = self.local_length
        return dist.all_to_all_single(recv_slot.reshape(-1), out_chunk.reshape(-1),
                                      output_split_sizes=[L * c * d] * self.world,
                                      input_split_sizes=[s * c * d for s in self.splits],
                                      group=self.group, async_op=async_op)

    def attention_packed(self, send: torch.Tensor, attn: Callable, overlap: bool = False) -> torch.Tensor:
        """Sequence-parallel attention on a pre-packed send buffer [chunks, world, L_r, c, 3, D]
        (what ops.qk_norm_rope_pack writes).  Per chunk: all-to-all, attention over the c
        local heads, reverse all-to-all into slot [ch] of the result
        [chunks, world, L_r, c, D], which ops.quantize_int8_rowwise_gathered (or
        `unpack_gathered`) reads in place.  With `overlap` the transfers run on a side stream:
        chunk i's attention overlaps chunk i+1's forward and chunk i-1's reverse transfer."""
        chunks, world, L, c, _, d = send.shape
        if world != self.world or L != self.local_length or chunks * c != self.local_heads:
            raise RuntimeError("send buffer does not match this sequence-parallel group")
        result = torch.empty((chunks, world, L, c, d), device=send.device, dtype=send.dtype)
        if overlap and send.is_cuda:
            main = torch.cuda.current_stream(send.device)
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=send.device)
            comm = self._comm_stream
            ready = torch.cuda.Event()
            ready.record(main)
            received = []
            with torch.cuda.stream(comm):
                comm.wait_event(ready)
                for ch in range(chunks):
                    recv, work = self.exchange_packed(send[ch], async_op=True)
                    work.wait()
                    done = torch.cuda.Event()
                    done.record(comm)
                    received.append((recv, done))
            for ch, (recv, done) in enumerate(received):
                main.wait_event(done)
                recv.record_stream(main)
                out = attn(*self.chunk_views(recv))           # [1,c,S,D] view of [1,S,c,D]
                out_ready = torch.cuda.Event()
                out_ready.record(main)
                with torch.cuda.stream(comm):
                    comm.wait_event(out_ready)
                    out.record_stream(comm)
                    self.reverse_into(out.transpose(1, 2).reshape(self.sequence, c, d), result[ch],
                                      async_op=True).wait()
            back = torch.cuda.Event()
            back.record(comm)
            main.wait_event(back)
            send.record_stream(comm)
            result.record_stream(comm)
        else:
            for ch in range(chunks):
                recv, _ = self.exchange_packed(send[ch])
                out = attn(*self.chunk_views(recv))
                self.reverse_into(out.transpose(1, 2).reshape(self.sequence, c, d), result[ch])
        return result

    @staticmethod
    def unpack_gathered(result: torch.Tensor) -> torch.Tensor:
        """[chunks, world, L, c, D] -> [L, H*D] with head h = (p*chunks + ch)*c + ci (a copy;
        the quantizer reads the gathered layout directly instead)."""
        chunks, world, L, c, d = result.shape
        return result.permute(2, 1, 0, 3, 4).reshape(L, world * chunks * c * d)

    # -- attention variants -------------------------------------------------------------
    def attention_baseline(self, qkv: torch.Tensor, attn: Callable) -> torch.Tensor:
        """Three all-to-alls, one attention over the local heads, reverse all-to-all.
        `attn(q,k,v)` maps [1,h,S,D] views to a [1,h,S,D] view of [1,S,h,D] storage."""
        parts = [self.sequence_to_heads(qkv[:, i]) for i in range(3)]
        q, k, v = (t.transpose(0, 1).unsqueeze(0) for t in parts)
        out = attn(q, k, v)
        return self.heads_to_sequence(out.transpose(1, 2).reshape(self.sequence, self.local_heads,
                                                                  self.dim))

    def attention_fused(self, qkv: torch.Tensor, attn: Callable, chunks: int = 1,
                        overlap: bool = False) -> torch.Tensor:
        """One packed all-to-all per head chunk; with `overlap` the all-to-alls run on a
        side stream and chunk i's attention overlaps chunk i+1's transfer."""
        hl = self.local_heads
        if hl % chunks:
            raise RuntimeError("chunk count must divide the local head count")
        step = hl // chunks
        bounds = [(i * step, (i + 1) * step) for i in range(chunks)]
        outputs = []
        if overlap and qkv.is_cuda:
            if self._comm_stream is None:
                self._comm_stream = torch.cuda.Stream(device=qkv.device)
            ready = torch.cuda.Event()
            ready.record(torch.cuda.current_stream(qkv.device))
            pending = []
            with torch.cuda.stream(self._comm_stream):
                self._comm_stream.wait_event(ready)
                for a, b in bounds:
                    item = self.pack_chunk(qkv, a, b, async_op=True)
                    done = torch.cuda.Event()
                    item[2].wait()          # orders the side stream after the collective
                    done.record(self._comm_stream)
                    pending.append((item, done))
            for (recv, send, _work), done in pending:
                torch.cuda.current_stream(qkv.device).wait_event(done)
                recv.record_stream(torch.cuda.current_stream(qkv.device))
                send.record_stream(self._comm_stream)
                outputs.append(attn(*self.chunk_views(recv)))
        else:
            for a, b in bounds:
                recv, _send, work = self.pack_chunk(qkv, a, b, async_op=False)
                outputs.append(attn(*self.chunk_views(recv)))
        # each output is a [1,c,S,D] view of [1,S,c,D] storage
        seq_major = [o.transpose(1, 2).reshape(self.sequence, -1, self.dim) for o in outputs]
        merged = seq_major[0] if len(seq_major) == 1 else torch.cat(seq_major, dim=1)
        return self.heads_to_sequence(merged)
