"""Ulysses layout transforms on two CPU ranks (gloo): uneven token splits, the
packed head-chunk all-to-all, the call order and layouts of the peer-store exchange (peer
memory emulated by collectives), and the agreement check of the overlap flag."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, seq, heads, flag_mismatch, result_dir):
    sys.path.insert(0, str(ROOT))
    import importlib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module("dcu-video-dit-turbo_b200")
        from oracle import ref_ops as ref
        if flag_mismatch:
            try:
                pkg.gates.agree_flag_across_ranks(rank == 0)
                outcome = "no error"
            except RuntimeError as exc:
                outcome = str(exc)
            Path(result_dir, f"r{rank}.txt").write_text(outcome)
            return
        pkg.gates.agree_flag_across_ranks(True)
        D = 8
        splits = pkg.ulysses.sequence_splits(seq, world)
        assert list(splits) == ref.ulysses_splits(seq, world)
        sp = pkg.ulysses.UlyssesSP(splits, heads, D)
        # every rank builds ALL shards from the same seed, so each can check its part
        g = torch.Generator().manual_seed(20260812)
        qkv_all = [torch.randint(-8, 9, (n, 3, heads, D), generator=g).to(torch.bfloat16) for n in splits]
        mine = qkv_all[rank]
        # plain transforms against the single-process model
        for part in range(3):
            got = sp.sequence_to_heads(mine[:, part].contiguous())
            want = ref.sequence_to_heads_all([t[:, part] for t in qkv_all])[rank]
            assert torch.equal(got, want)
            back = sp.heads_to_sequence(got)
            assert torch.equal(back, mine[:, part])
        # packed head chunks: [S, c, 3, D] must hold the same q/k/v as three separate transforms
        hl = heads // world
        for chunks in (1, hl):
            step = hl // chunks
            for c in range(chunks):
                recv, _, _ = sp.pack_chunk(mine, c * step, (c + 1) * step, async_op=False)
                q, k, v = sp.chunk_views(recv)
                assert tuple(q.stride()[1:]) == (3 * D, step * 3 * D, 1)
                for part, t in enumerate((q, k, v)):
                    want = ref.sequence_to_heads_all([x[:, part] for x in qkv_all])[rank]
                    assert torch.equal(t[0].transpose(0, 1), want[:, c * step:(c + 1) * step])
        # attention variants with a stand-in "attention" (elementwise, layout-preserving):
        # baseline and fused chunked paths must agree bitwise and land in token order
        attn = lambda q, k, v: (q + k * 2 + v * 4).transpose(1, 2).contiguous().transpose(1, 2)
        base = sp.attention_baseline(mine, attn)
        want = (mine[:, 0] + mine[:, 1] * 2 + mine[:, 2] * 4)
        assert torch.equal(base, want)
        for chunks in (1, hl):
            assert torch.equal(sp.attention_fused(mine, attn, chunks=chunks, overlap=False), want)
        # pre-packed exchange: the send buffer is built destination-major up front (what the
        # fused norm+rotary+pack kernel writes) and the result stays in the reverse
        # all-to-all's layout (what the gathered quantizer reads)
        for chunks in (1, hl):
            send = ref.pack_send(mine, world, chunks)
            for ch in range(chunks):
                recv, _ = sp.exchange_packed(send[ch])
                legacy, _, _ = sp.pack_chunk(mine, ch * (hl // chunks), (ch + 1) * (hl // chunks), async_op=False)
                assert torch.equal(recv, legacy)
            result = sp.attention_packed(send, attn, overlap=False)
            assert tuple(result.shape) == (chunks, world, splits[rank], hl // chunks, D)
            assert torch.equal(ref.unpack_gathered(result), want.reshape(splits[rank], heads * D))
            assert torch.equal(sp.unpack_gathered(result), want.reshape(splits[rank], heads * D))
        # the peer-store form of the exchange, with the peers' memory emulated by collectives: the
        # "scatter kernel" delivers what pack + all-to-all delivers, the "push kernel" moves the
        # byte ranges of peer.push_plan; attention_peer must order scatter, barrier, attention,
        # push, barrier and return the gathered layout of the collective path
        log = []

        class EmulatedPeer:
            def __init__(self):
                self.recv = torch.zeros((1, sp.sequence, hl, 3, D), dtype=torch.bfloat16)
                self.result = torch.zeros((1, world, splits[rank], hl, D), dtype=torch.bfloat16)
                self.recv_buffer = type("Buffer", (), {"table": "receive-buffer table"})()

            def barrier(self):
                log.append("barrier")
                dist.barrier()

            def push(self, rows):
                log.append("push")
                assert rows.shape == (sp.sequence, hl, D) and rows.is_contiguous()
                flat = rows.reshape(-1).view(torch.int16)
                outgoing = [None] * world
                for peer_rank, src_off, dst_off, nbytes in pkg.peer.push_plan(splits, rank, hl, D):
                    assert dst_off == rank * splits[peer_rank] * hl * D * 2
                    outgoing[peer_rank] = flat[src_off // 2:(src_off + nbytes) // 2].clone()
                everything = [None] * world        # every rank's outgoing ranges (stands in for the peer stores)
                dist.all_gather_object(everything, outgoing)
                for src in range(world):
                    self.result.view(torch.int16).view(world, -1)[src] = everything[src][rank]

        def scatter(table, row0, sequence):
            log.append("scatter")
            assert table == "receive-buffer table" and row0 == sum(splits[:rank]) and sequence == seq
            send = ref.pack_send(mine, world, 1)[0]                       # [world, L, hl, 3, D]
            everything = [None] * world
            dist.all_gather_object(everything, send)
            start = 0
            for src in range(world):
                sp.peer.recv[0, start:start + splits[src]] = everything[src][rank]
                start += splits[src]

        def logged_attn(q, k, v):
            log.append("attention")
            return attn(q, k, v)

        sp.peer = EmulatedPeer()
        gathered = sp.attention_peer(scatter, logged_attn)
        assert log == ["scatter", "barrier", "attention", "push", "barrier"], log
        assert gathered is sp.peer.result
        assert torch.equal(ref.unpack_gathered(gathered), want.reshape(splits[rank], heads * D))
        assert torch.equal(gathered, sp.attention_packed(ref.pack_send(mine, world, 1), attn, overlap=False))
        sp.peer = None
        try:
            sp.attention_peer(scatter, attn)
            raise AssertionError("attention_peer without peer buffers must raise")
        except RuntimeError as exc:
            assert "enable_peer_exchange" in str(exc)
        Path(result_dir, f"r{rank}.txt").write_text("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("seq,heads", [(23, 4), (30, 6)])
def test_two_rank_layouts(tmp_path, seq, heads):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, seq, heads, False, str(tmp_path)), nprocs=2, join=True)
    assert [Path(tmp_path, f"r{r}.txt").read_text() for r in range(2)] == ["ok", "ok"]


def test_flag_disagreement_raises_on_every_rank(tmp_path):
    port = _free_port()
    mp.spawn(_worker, args=(2, port, 16, 4, True, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        assert "differs between distributed ranks" in Path(tmp_path, f"r{r}.txt").read_text()
