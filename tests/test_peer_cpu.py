"""Host side of the peer-memory exchange without a GPU: the push plan (which bytes of a rank's
attention output go where in which owner's gathered buffer) replayed on plain byte arrays must
produce exactly what the reverse all-to-all of the collective path delivers
(ulysses.UlyssesSP.reverse_into; the reference's layout is
benchmarks/bench_sp_head_chunk_overlap.py:104-118), for even and ragged token splits."""
import numpy as np
import pytest
import torch


@pytest.mark.parametrize("world,seq", [(2, 10), (2, 11), (4, 23), (8, 64), (8, 67), (8, 5), (3, 7)])
def test_push_plan_replayed_on_bytes_equals_the_reverse_all_to_all(pkg, ref, world, seq):
    heads, dim = 24, 16
    hl = heads // world
    splits = pkg.ulysses.sequence_splits(seq, world)
    rng = np.random.default_rng(world * 100 + seq)
    outs = [rng.integers(-30000, 30000, size=(seq, hl, dim), dtype=np.int16) for _ in range(world)]
    gathered = [np.zeros((world, splits[p], hl, dim), dtype=np.int16) for p in range(world)]
    for r in range(world):
        plan = pkg.peer.push_plan(splits, r, hl, dim)
        assert [p for p, *_ in plan] == [(r + 1 + i) % world for i in range(world)]
        src = outs[r].reshape(-1).view(np.uint8)
        for p, src_off, dst_off, nbytes in plan:
            assert src_off % 16 == 0 and dst_off % 16 == 0 and nbytes % 16 == 0
            dst = gathered[p].reshape(-1).view(np.uint8)
            assert dst_off + nbytes <= dst.size and src_off + nbytes <= src.size
            dst[dst_off:dst_off + nbytes] = src[src_off:src_off + nbytes]
    row0 = 0
    for p in range(world):
        rows = slice(row0, row0 + splits[p])
        for r in range(world):
            assert np.array_equal(gathered[p][r], outs[r][rows])
        # and through the oracle's unpack: token-major rows with heads in global order
        want = np.concatenate([outs[r][rows] for r in range(world)], axis=1).reshape(splits[p], heads * dim)
        got = ref.unpack_gathered(torch.from_numpy(gathered[p][None].copy())).numpy()
        assert np.array_equal(got, want)
        row0 += splits[p]


def test_peer_exchange_needs_a_cuda_device(pkg):
    with pytest.raises(RuntimeError, match="CUDA device memory"):
        pkg.peer.PeerBuffer(64, torch.device("cpu"))


def test_interleave_gate_up_is_a_permutation_in_groups_of_64(pkg):
    """Host-side weight preparation for the SwiGLU epilogue (pure tensor indexing, no kernel):
    rows [128k, 128k+64) of the result are gate rows [64k, 64k+64), rows [128k+64, 128k+128) the
    matching up rows, for weights, scales and biases alike."""
    ops = pkg.ops
    f = 192
    w = torch.arange(2 * f * 5).view(2 * f, 5)
    il = ops.interleave_gate_up(w)
    assert il.shape == w.shape and il.is_contiguous()
    for k in range(f // 64):
        assert torch.equal(il[128 * k:128 * k + 64], w[64 * k:64 * k + 64])                  # gate rows
        assert torch.equal(il[128 * k + 64:128 * k + 128], w[f + 64 * k:f + 64 * k + 64])    # up rows
    v = torch.arange(2 * f)
    assert torch.equal(ops.interleave_gate_up(v), ops.interleave_gate_up(v.view(-1, 1)).view(-1))
    assert sorted(ops.interleave_gate_up(v).tolist()) == v.tolist()
    with pytest.raises(RuntimeError, match="multiple of 128"):
        ops.interleave_gate_up(torch.zeros(2 * 96))
