"""The peer-memory exchange kernels on ONE GPU: the ranks of a sequence-parallel group are
emulated as buffers of the same device (every "peer" address is local), so the addressing of
ops.qk_norm_rope_scatter and of the push plan is checked bit for bit against the layouts of
the all-to-all path (oracle: ref_ops.pack_send / unpack_gathered, the reference's
benchmarks/bench_sp_head_chunk_overlap.py:140-164 and :83-118) without a second GPU.  The
IPC mapping itself needs two processes on two GPUs: tests/test_gpu_multi.py."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
H, D = 24, 128


def _splits(pkg, seq, world):
    return pkg.ulysses.sequence_splits(seq, world)


@pytest.mark.parametrize("world,chunks,seq", [(2, 1, 1001), (4, 1, 777), (8, 1, 1030), (3, 2, 515), (8, 3, 64), (2, 1, 1)])
def test_rope_scatter_fills_every_rank_like_pack_plus_all_to_all(cuda_pkg, ref, world, chunks, seq):
    ops = cuda_pkg.ops
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(100 + world)
    qkv = torch.randn((seq, 3, H, D), generator=g).to(torch.bfloat16)
    qw = (1.0 + 0.02 * torch.randn((D,), generator=g)).to(torch.bfloat16)
    kw = (1.0 + 0.02 * torch.randn((D,), generator=g)).to(torch.bfloat16)
    cos, sin = cuda_pkg.block.rope_tables(cuda_pkg.block.grid_positions(seq))
    # what every rank must end up holding: the in-place kernel on all rows, then the heads of
    # rank p, chunk ch, as [S, c, 3, D]
    done = ops.qk_norm_rope_(qkv.clone().to(dev), qw.to(dev), kw.to(dev), cos.to(dev), sin.to(dev)).cpu()
    c = H // (world * chunks)
    splits = _splits(cuda_pkg, seq, world)
    recv = [torch.full((chunks, seq, c, 3, D), 7.0, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    table = (ctypes.c_void_p * world)(*[t.data_ptr() for t in recv])
    row0 = 0
    for r in range(world):
        rows = slice(row0, row0 + splits[r])
        ops.qk_norm_rope_scatter(qkv[rows].contiguous().to(dev), qw.to(dev), kw.to(dev),
                                 cos[rows].contiguous().to(dev), sin[rows].contiguous().to(dev),
                                 table, world, row0, seq, chunks=chunks)
        row0 += splits[r]
    torch.cuda.synchronize()
    ops.check_device_status(dev)
    for p in range(world):
        for ch in range(chunks):
            h0 = (p * chunks + ch) * c
            want = done[:, :, h0:h0 + c].permute(0, 2, 1, 3)          # [S, c, 3, D]
            assert torch.equal(recv[p][ch].cpu().view(torch.int16), want.contiguous().view(torch.int16)), (p, ch)
    # and it is what the packing kernel + an all-to-all would have delivered
    row0 = 0
    for r in range(world):
        rows = slice(row0, row0 + splits[r])
        send = ops.qk_norm_rope_pack(qkv[rows].contiguous().to(dev), qw.to(dev), kw.to(dev),
                                     cos[rows].contiguous().to(dev), sin[rows].contiguous().to(dev), world, chunks)
        for p in range(world):
            for ch in range(chunks):
                assert torch.equal(recv[p][ch, rows], send[ch, p])
        row0 += splits[r]


@pytest.mark.parametrize("world,seq", [(2, 1001), (4, 23), (8, 1030), (8, 5)])
def test_push_plan_and_copy_segments_gather_like_the_reverse_all_to_all(cuda_pkg, ref, world, seq):
    ops, peer = cuda_pkg.ops, cuda_pkg.peer
    dev = torch.device("cuda:0")
    hl = H // world
    splits = _splits(cuda_pkg, seq, world)
    g = torch.Generator().manual_seed(7 * world + seq)
    outs = [torch.randn((seq, hl, D), generator=g).to(torch.bfloat16).to(dev) for _ in range(world)]
    result = [torch.full((1, world, splits[p], hl, D), 3.0, dtype=torch.bfloat16, device=dev) for p in range(world)]
    for r in range(world):
        plan = peer.push_plan(splits, r, hl, D)
        n = len(plan)
        assert sorted(p for p, *_ in plan) == list(range(world)) and plan[-1][0] == r
        src = (ctypes.c_void_p * n)()
        dst = (ctypes.c_void_p * n)(*[result[p].data_ptr() + off for (p, _s, off, _n) in plan])
        nbytes = (ctypes.c_int64 * n)(*[nb for (*_x, nb) in plan])
        ops.copy_segments(outs[r], [s for (_p, s, _d, _n) in plan], src, dst, nbytes, n,
                          sum(nb for (*_x, nb) in plan))
    torch.cuda.synchronize()
    row0 = 0
    for p in range(world):
        rows = slice(row0, row0 + splits[p])
        for r in range(world):
            assert torch.equal(result[p][0, r], outs[r][rows]), (p, r)
        # head order of the gathered layout: rank-major
        if splits[p]:
            want = torch.cat([outs[r][rows] for r in range(world)], dim=1).reshape(splits[p], H * D)
            assert torch.equal(ref.unpack_gathered(result[p].cpu()), want.cpu())
        row0 += splits[p]


def test_copy_segments_tail_sizes_and_refusals(cuda_pkg):
    ops = cuda_pkg.ops
    lib = cuda_pkg._lib.load()
    dev = torch.device("cuda:0")
    for nbytes in (16, 48, 16 * 1023, 16 * (4 * 256 * 3 + 5), 1 << 22):
        src = torch.randint(0, 255, (nbytes,), dtype=torch.uint8, device=dev)
        dst = torch.zeros((nbytes + 32,), dtype=torch.uint8, device=dev)
        tab_s, tab_d = (ctypes.c_void_p * 1)(), (ctypes.c_void_p * 1)(dst.data_ptr() + 16)
        ops.copy_segments(src, [0], tab_s, tab_d, (ctypes.c_int64 * 1)(nbytes), 1, nbytes)
        torch.cuda.synchronize()
        assert torch.equal(dst[16:16 + nbytes], src) and int(dst[:16].sum()) == 0 and int(dst[-16:].sum()) == 0
    P = ctypes.c_void_p
    one = (P * 1)(0x1000)
    assert lib.b2_copy_segments(one, one, (ctypes.c_int64 * 1)(24), 1, None) == 2       # not a multiple of 16
    assert lib.b2_copy_segments(one, (P * 1)(0x1008), (ctypes.c_int64 * 1)(32), 1, None) == 3
    assert lib.b2_copy_segments(one, one, (ctypes.c_int64 * 1)(32), 9, None) == 2
    with pytest.raises(RuntimeError, match="outside the source"):
        ops.copy_segments(torch.zeros(64, dtype=torch.uint8, device=dev), [32], (P * 1)(), one,
                          (ctypes.c_int64 * 1)(64), 1, 64)


def test_peer_buffer_allocation_export_and_view(cuda_pkg):
    """b2_peer_alloc / export / free on one device, and the zero-copy tensor view of it."""
    lib = cuda_pkg._lib.load()
    peer = cuda_pkg.peer
    ptr = ctypes.c_void_p()
    cuda_pkg._lib.check(lib.b2_peer_alloc(1 << 20, ctypes.byref(ptr)), "b2_peer_alloc")
    try:
        handle = ctypes.create_string_buffer(peer.HANDLE_BYTES)
        cuda_pkg._lib.check(lib.b2_peer_export(ptr.value, handle, peer.HANDLE_BYTES), "b2_peer_export")
        assert any(handle.raw)
        assert lib.b2_peer_export(ptr.value, handle, 8) == 2
        view = torch.as_tensor(peer._Span(ptr.value, 1 << 20, None), device="cuda:0")
        assert view.data_ptr() == ptr.value and int(view.sum()) == 0       # zero filled, not copied
        view.view(torch.bfloat16)[:8] = 1.5
        torch.cuda.synchronize()
        again = torch.as_tensor(peer._Span(ptr.value, 16, None), device="cuda:0").view(torch.bfloat16)
        assert again.tolist() == [1.5] * 8
        del view, again
    finally:
        torch.cuda.synchronize()
        cuda_pkg._lib.check(lib.b2_peer_free(ptr.value), "b2_peer_free")
    assert lib.b2_peer_alloc(0, ctypes.byref(ptr)) == 2
