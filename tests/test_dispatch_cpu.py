"""Launcher-level integration on the host: linear dispatch on the quantized weight class,
run-time toggles by signal, and the job digest agreed between ranks (gloo)."""
import hashlib
import json
import os
import signal
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def pkg():
    import importlib
    sys.path.insert(0, str(ROOT))
    return importlib.import_module("dcu-video-dit-turbo_b200")


def test_cpu_weight_falls_back_to_the_original_handler_and_is_counted(pkg):
    """On a CPU tensor the dispatch must refuse (wrong architecture) and hand the call to
    the original handler: the dequantized bf16 linear by default, or a registered one."""
    g = torch.Generator().manual_seed(3)
    w = (torch.randn((3072, 3072), generator=g) * 0.02).to(torch.bfloat16)
    x = torch.randn((5, 3072), generator=g).to(torch.bfloat16)
    bias = torch.randn((3072,), generator=g).to(torch.bfloat16)
    d = pkg.dispatch.LinearDispatch(gates=pkg.gates.Gates.all_on())
    qw = pkg.dispatch.quantize_weight(w, dispatch=d)
    assert tuple(qw.shape) == (3072, 3072) and qw.dtype == torch.bfloat16
    assert qw.qdata.dtype == torch.int8 and int(qw.qdata.abs().max()) == 127
    from oracle import ref_ops as ref
    wq_ref, ws_ref = ref.quantize_weight_per_channel(w)
    assert torch.equal(qw.qdata, wq_ref) and torch.equal(qw.scale, ws_ref)
    assert d.eligibility(x, qw) == "weight_shape_or_arch"
    with pytest.raises(RuntimeError, match="no original handler"):
        torch.nn.functional.linear(x, qw, bias)
    d.fallbacks.clear()
    d.register_original_handler(pkg.dispatch.dequantized_linear)
    y = torch.nn.functional.linear(x, qw, bias)
    assert torch.equal(y, torch.nn.functional.linear(x, qw.dequantize(), bias))
    assert d.summary() == {"enabled": True, "routed": 0, "fallbacks": {"weight_shape_or_arch": 1}}
    seen = []
    d.register_original_handler(lambda inp, weight, b: seen.append(tuple(weight.shape)) or inp)
    assert torch.nn.functional.linear(x, qw) is x and seen == [(3072, 3072)]
    # refusal order: disabled first, then transposed
    d.set_enabled(False)
    assert d.eligibility(x, qw) == "disabled"
    d.set_enabled(True)
    qt = pkg.dispatch.Int8Weight(qw.qdata, qw.scale, transposed=True, dispatch=d)
    assert d.eligibility(x, qt) == "transposed"
    assert d.eligibility(qw, qw) == "quantized_input"
    with pytest.raises(NotImplementedError):
        qw + 1


def test_signals_toggle_the_route_in_a_running_process(pkg):
    d = pkg.dispatch.LinearDispatch()
    prev = d.install_signal_toggles()
    try:
        os.kill(os.getpid(), signal.SIGUSR2)
        assert d.enabled is False
        os.kill(os.getpid(), signal.SIGUSR1)
        assert d.enabled is True
    finally:
        signal.signal(signal.SIGUSR1, prev[0])
        signal.signal(signal.SIGUSR2, prev[1])


def test_job_digest_is_the_sha256_of_the_canonical_contract(pkg):
    prompt = {"7": {"class_type": "BasicGuider", "inputs": {"model": ["3", 0]}}, "3": {"class_type": "Loader"}}
    hashes = {"positive": "ab" * 32}
    want = hashlib.sha256(json.dumps({"prompt": prompt, "conditioning_inputs": hashes}, ensure_ascii=False,
                                     sort_keys=True, separators=(",", ":")).encode("utf-8")).hexdigest()
    assert pkg.dispatch.job_digest(prompt, hashes) == want
    reordered = {"3": {"class_type": "Loader"}, "7": {"inputs": {"model": ["3", 0]}, "class_type": "BasicGuider"}}
    assert pkg.dispatch.job_digest(reordered, hashes) == want          # key order does not matter
    assert pkg.dispatch.job_digest(prompt, hashes, seed=1) != pkg.dispatch.job_digest(prompt, hashes, seed=2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _digest_worker(rank, world, port, same, result_dir):
    import importlib
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module("dcu-video-dit-turbo_b200")
        digest = pkg.dispatch.job_digest({"1": {"seed": 0 if same else rank}})
        try:
            pkg.dispatch.agree_digest_across_ranks(digest)
            outcome = "agreed"
        except RuntimeError as exc:
            outcome = str(exc)
        Path(result_dir, f"r{rank}.txt").write_text(outcome)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("same", [True, False])
def test_ranks_must_hold_the_same_job_digest(tmp_path, same):
    mp.spawn(_digest_worker, args=(2, _free_port(), same, str(tmp_path)), nprocs=2, join=True)
    texts = [Path(tmp_path, f"r{r}.txt").read_text() for r in range(2)]
    if same:
        assert texts == ["agreed", "agreed"]
    else:
        assert all("job digest differs between distributed ranks" in t for t in texts)
