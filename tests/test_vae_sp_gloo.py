"""Temporal-chunk parallel VAE decode on CPU ranks (gloo) with a stand-in decoder: the clip
assembled from the ranks' packets is bitwise the sequential one, for even and uneven chunk
splits, and the validate mode catches a rank that decodes something else."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]
CHUNK, UP, OVER = 3, 4, 2          # latent frames per chunk, frames per latent frame, overlap frames


def _decode_parts(z, index, poison_rank=None):
    """Stand-in decoder: chunk `index` of latents [1,C,T,H,W] -> (main, overlap) frames; the
    first chunk has extra leading frames, like a decoder with frame pre-padding."""
    zc = z[:, :, index * CHUNK:(index + 1) * CHUNK]
    frames = zc.repeat_interleave(UP, dim=2) * (index + 1) + index
    if index == 0:
        frames = torch.cat((frames[:, :, :1] - 1, frames), dim=2)
    if poison_rank is not None and dist.is_initialized() and dist.get_rank() == poison_rank:
        frames = frames + 1
    return frames[:, :, :-OVER].contiguous(), frames[:, :, -OVER:].contiguous()


def _blend(prev_overlap, main, n):
    w = torch.linspace(0, 1, n).view(1, 1, n, 1, 1)
    out = main.clone()
    out[:, :, :n] = prev_overlap * (1 - w) + main[:, :, :n] * w
    return out


def _frames(num_chunks):
    # every chunk contributes its main frames, the last one its overlap as well
    return num_chunks * (CHUNK * UP - OVER) + 1 + OVER


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, num_chunks, poison, result_dir):
    import importlib
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module("dcu-video-dit-turbo_b200")
        g = torch.Generator().manual_seed(3)
        z = torch.randn((1, 2, num_chunks * CHUNK, 3, 5), generator=g)
        if rank != 0:
            z = torch.zeros_like(z)                       # only rank 0 holds the latents
        dec = pkg.vae_sp.TemporalChunkDecode(num_chunks, _frames(num_chunks), OVER, validate=poison)
        parts = (lambda zz, i: _decode_parts(zz, i, poison_rank=1)) if poison else _decode_parts
        try:
            out = dec.decode(z, parts, _blend)
            if rank == 0:
                g = torch.Generator().manual_seed(3)
                z0 = torch.randn((1, 2, num_chunks * CHUNK, 3, 5), generator=g)
                want = dec.decode_single(z0, _decode_parts, _blend)
                outcome = "equal" if torch.equal(out, want) and out.shape[2] == _frames(num_chunks) else "differs"
            else:
                outcome = "none" if out is None else "unexpected"
        except RuntimeError as exc:
            outcome = str(exc)
        Path(result_dir, f"r{rank}.txt").write_text(outcome)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,num_chunks", [(2, 7), (2, 4), (3, 7)])
def test_parallel_decode_is_bitwise_the_sequential_one(tmp_path, world, num_chunks):
    mp.spawn(_worker, args=(world, _free_port(), num_chunks, False, str(tmp_path)), nprocs=world, join=True)
    texts = [Path(tmp_path, f"r{r}.txt").read_text() for r in range(world)]
    assert texts == ["equal"] + ["none"] * (world - 1)


def test_validate_mode_rejects_a_rank_that_decodes_differently(tmp_path):
    mp.spawn(_worker, args=(2, _free_port(), 5, True, str(tmp_path)), nprocs=2, join=True)
    assert "is not bitwise exact" in Path(tmp_path, "r0.txt").read_text()


def test_chunk_ranges_match_the_reference_cut():
    import importlib
    sys.path.insert(0, str(ROOT))
    vs = importlib.import_module("dcu-video-dit-turbo_b200").vae_sp
    assert [list(r)[0] for r in vs.chunk_ranges(21, 2)] == [0, 11] and len(vs.chunk_ranges(21, 2)[1]) == 10
    assert [len(r) for r in vs.chunk_ranges(7, 3)] == [3, 2, 2]
    assert [len(r) for r in vs.chunk_ranges(2, 4)] == [1, 1, 0, 0]
