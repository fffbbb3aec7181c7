"""Device buffers that the other ranks of one machine can write into, and the plan of the
sequence-parallel exchange carried over them.

`PeerBuffer` allocates one buffer per rank through the C ABI (b2_peer_alloc), exchanges the
CUDA IPC handles over the process group and maps every peer's buffer into this process, so
that this rank's kernels can store straight into memory of the rank that will read the data
(ordinary stores over NVLink; no kernel waits on another GPU and no library kernel is handed
a peer pointer).  `PeerExchange` holds the two buffers of a Ulysses group: the receive buffer
of the forward direction, bf16 [1, S, H/P, 3, D], which ops.qk_norm_rope_scatter of every rank
fills, and the gathered buffer of the reverse direction, bf16 [1, P, L_r, H/P, D], which
ops.copy_segments of every rank fills and ops.quantize_int8_rowwise_gathered reads.  The
byte layouts are those of the all-to-all path in ulysses.py (the reference's model:
benchmarks/bench_sp_head_chunk_overlap.py:140-164 and :83-118), so both transports give the
same bits.

Ordering between ranks is one small all-reduce on the compute stream after each direction's
writes: it cannot complete on any rank before every rank has reached it, i.e. before every
rank's preceding kernel has finished.  With the whole exchange on ONE stream that also
covers reuse of the two buffers by the next step (see `UlyssesSP.attention_peer`).
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch
import torch.distributed as dist

from . import _lib

HANDLE_BYTES = 64


class _Span:
    """A raw device address range as an object torch can wrap without copying."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2}


def push_plan(splits: Sequence[int], rank: int, local_heads: int, dim: int, itemsize: int = 2):
    """Reverse direction, as (peer, src_offset, dst_offset, nbytes) per peer, in bytes.

    This rank holds the attention output [S, c, D] of its c = H/P heads for all S rows; rows
    [row0_p, row0_p + L_p) belong to rank p and go to slot [rank] of p's gathered buffer
    [P, L_p, c, D].  Peers are listed starting after this rank, so that at any moment the
    ranks write to different destinations."""
    world = len(splits)
    width = local_heads * dim * itemsize
    row0 = [sum(splits[:p]) for p in range(world)]
    plan = []
    for i in range(world):
        p = (rank + 1 + i) % world
        plan.append((p, row0[p] * width, rank * splits[p] * width, splits[p] * width))
    return plan


class PeerBuffer:
    """`nbytes` of zero-filled device memory on every rank of `group`, each rank's buffer
    mapped in every process.  `ptrs[p]` is rank p's buffer as addressed from here;
    `table` is the same as a C array for the ABI.  Collective: every rank must construct it
    at the same point (the handles travel through all_gather_object)."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        if device.type != "cuda":
            raise RuntimeError("peer buffers live in CUDA device memory")
        self.lib = _lib.load()
        self.device = device
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.nbytes = int(nbytes)
        self._opened: list[int] = []
        self._local = 0
        # A rank that fails here must not leave the others waiting in a collective: every
        # rank goes through the same two collectives and all of them raise if one failed.
        handle = ctypes.create_string_buffer(HANDLE_BYTES)
        failure = None
        self.ptrs: list[int] = []
        self.sizes: list[int] = []
        with torch.cuda.device(device):
            try:
                out = ctypes.c_void_p()
                _lib.check(self.lib.b2_peer_alloc(self.nbytes, ctypes.byref(out)), "b2_peer_alloc")
                self._local = out.value
                _lib.check(self.lib.b2_peer_export(self._local, handle, HANDLE_BYTES), "b2_peer_export")
            except RuntimeError as exc:
                failure = exc
            gathered: list = [None] * self.world
            dist.all_gather_object(gathered, (self.rank, self.nbytes, handle.raw, failure is None), group=group)
            if failure is None and all(item[3] for item in gathered):
                try:
                    for p, (peer_rank, peer_bytes, raw, _ok) in enumerate(gathered):
                        if peer_rank != p:
                            raise RuntimeError("peer handles arrived out of rank order")
                        self.sizes.append(peer_bytes)
                        if p == self.rank:
                            self.ptrs.append(self._local)
                            continue
                        mapped = ctypes.c_void_p()
                        _lib.check(self.lib.b2_peer_open(raw, HANDLE_BYTES, ctypes.byref(mapped)), "b2_peer_open")
                        self._opened.append(mapped.value)
                        self.ptrs.append(mapped.value)
                except RuntimeError as exc:
                    failure = exc
            elif failure is None:
                failure = RuntimeError("another rank could not allocate or export its buffer")
            agreed = torch.tensor([0 if failure is not None else 1], dtype=torch.int32, device=device)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN, group=group)
            if int(agreed.item()) == 0:
                for ptr in self._opened:
                    self.lib.b2_peer_close(ptr)
                self._opened = []
                dist.barrier(group=group)
                if self._local:
                    self.lib.b2_peer_free(self._local)
                    self._local = 0
                raise RuntimeError(f"peer buffer set-up failed on at least one rank"
                                   f"{': ' + str(failure) if failure is not None else ''}")
        self.table = (ctypes.c_void_p * self.world)(*self.ptrs)

    def tensor(self, dtype: torch.dtype, shape: Sequence[int]) -> torch.Tensor:
        """The local buffer as a tensor (no copy).  Keep this object alive while it is used."""
        need = torch.empty((), dtype=dtype).element_size()
        for n in shape:
            need *= int(n)
        if need > self.nbytes:
            raise RuntimeError(f"a {tuple(shape)} {dtype} tensor needs {need} bytes, the buffer has {self.nbytes}")
        if need == 0:
            return torch.empty(tuple(shape), dtype=dtype, device=self.device)
        flat = torch.as_tensor(_Span(self._local, need, self), device=self.device)
        return flat.view(dtype).view(*shape)

    def close(self) -> None:
        """Unmap the peers' buffers, wait for every rank to have done so, free the local one."""
        if not self._local:
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            for ptr in self._opened:
                _lib.check(self.lib.b2_peer_close(ptr), "b2_peer_close")
            self._opened = []
            dist.barrier(group=self.group)
            _lib.check(self.lib.b2_peer_free(self._local), "b2_peer_free")
        self._local = 0


class PeerExchange:
    """The two peer buffers of one Ulysses group and the per-step calls on them."""

    def __init__(self, splits: Sequence[int], heads: int, dim: int, device: torch.device, group=None):
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 8:
            raise RuntimeError("the peer exchange addresses at most 8 ranks")
        if heads % self.world:
            raise RuntimeError("world size must divide the head count")
        self.splits = tuple(int(s) for s in splits)
        self.sequence = sum(self.splits)
        self.local_length = self.splits[self.rank]
        self.row0 = sum(self.splits[:self.rank])
        self.local_heads = heads // self.world
        self.dim = dim
        hl, d, S, L = self.local_heads, dim, self.sequence, self.local_length
        self.recv_buffer = PeerBuffer(max(S * hl * 3 * d * 2, 16), device, group)
        self.result_buffer = PeerBuffer(max(self.world * L * hl * d * 2, 16), device, group)
        self.recv = self.recv_buffer.tensor(torch.bfloat16, (1, S, hl, 3, d))
        self.result = self.result_buffer.tensor(torch.bfloat16, (1, self.world, L, hl, d))
        self._token = torch.zeros(1, dtype=torch.int32, device=device)
        plan = push_plan(self.splits, self.rank, hl, d)
        n = len(plan)
        self._src_offsets = [src for (_p, src, _dst, _n) in plan]
        self._src = (ctypes.c_void_p * n)()
        self._dst = (ctypes.c_void_p * n)(*[self.result_buffer.ptrs[p] + dst for (p, _s, dst, _n) in plan])
        self._bytes = (ctypes.c_int64 * n)(*[nb for (_p, _s, _d, nb) in plan])
        self._segments = n
        self.push_bytes = sum(nb for (_p, _s, _d, nb) in plan)
        self.push_remote_bytes = sum(nb for (p, _s, _d, nb) in plan if p != self.rank)

    def barrier(self) -> None:
        """Every rank's preceding work on the current stream has finished once this has."""
        dist.all_reduce(self._token, group=self.group)

    def push(self, out_rows: torch.Tensor) -> None:
        """out_rows bf16 [S, H/P, D] contiguous: every owner's rows into its gathered buffer."""
        from . import ops
        ops.copy_segments(out_rows, self._src_offsets, self._src, self._dst, self._bytes, self._segments,
                          self.push_bytes, self.push_remote_bytes)

    def close(self) -> None:
        self.recv = self.result = None
        self.recv_buffer.close()
        self.result_buffer.close()
