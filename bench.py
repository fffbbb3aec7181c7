#!/usr/bin/env python
"""Headline benchmark: one random-init DiT transformer block, device-timed.

    python bench.py --gpus N --steps K --warmup W [--tokens T] [--impl reference]

A step is one forward pass of the block (adaLN -> INT8 QKV GEMM -> QK RMSNorm +
3-D RoPE -> bf16 flash attention -> INT8 out-proj -> adaLN -> SwiGLU FFN) over a
joint token stream of T tokens (default 109099 = 1344x768, 15 s of video+audio;
hidden 3072, 24 heads x 128, FFN 8192), synthetic activations ~N(0,1) and weights
~N(0,0.02) quantised per output channel.  With N > 1 (torchrun, one rank per GPU)
the SAME T tokens are sharded across ranks (Ulysses: token shards for the linears,
head shards for attention, NCCL all-to-all per head chunk), i.e. strong scaling.

Prints ONE JSON line on rank 0.  `value` is the block time in ms (max over ranks),
`e2e` the same through the public API with the host->device copy of the input
shard and the device->host copy of the output inside the timed region.
`--impl reference` times the CPU restatement of the reference's PyTorch path on a
bounded sample of the same workload on the host cores.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

HIDDEN, HEADS, HEAD_DIM, FFN = 3072, 24, 128, 8192
METRIC = "dit_block_ms"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--tokens", type=int, default=109099)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--head-chunks", type=int, default=0, help="0 = auto")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fuse-residual", action="store_true",
                    help="gated residuals as their own kernel instead of in the GEMM epilogue")
    ap.add_argument("--no-graph", action="store_true", help="single GPU: launch the kernels one by one")
    ap.add_argument("--kernel", default=None,
                    choices=["flash", "gemm_qkv", "gemm_fc1", "gemm_c1", "quant", "swiglu", "mod", "ln_quant", "rope_pack", "quant_gathered", "gemm_out_residual", "gemm_fc2", "gemm_fc2_residual", "frames_u8",
                             "epilogue", "gate", "rope"],
                    help="time ONE kernel alone on the block's shapes instead of the block")
    ap.add_argument("--cpu-seconds", type=float, default=20.0)
    return ap.parse_args()


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"],
                "bf16_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi during the timed region."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------
# CPU arm: the oracle's PyTorch restatement of the reference path on the host cores
# --------------------------------------------------------------------------------------

def cpu_block_ms(tokens: int, budget_s: float) -> dict:
    """Time the reference's PyTorch-CPU path on a bounded sample and scale to one block.

    Row-local ops (LayerNorm+modulation, quantizer, INT8 GEMM, epilogue, swiglu, RoPE,
    residual) run on a sample of `rows` token rows and scale by tokens/rows; attention
    runs `qrows` query rows of ONE head against ALL keys and scales by
    (tokens/qrows) x heads."""
    import torch
    from oracle import ref_ops as ref

    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(0)
    pkg = importlib.import_module("dcu-video-dit-turbo_b200")
    p = pkg.block.make_block_params(HIDDEN, HEADS, HEAD_DIM, FFN, seed=0, device="cpu")
    rows = 512
    x = torch.randn((rows, HIDDEN), generator=g).to(torch.bfloat16)
    cos, sin = ref.rope_tables(pkg.block.grid_positions(rows))

    def rowlocal():
        h = ref.mod_scale_shift(ref.layer_norm_noaffine(x), p["scale1"], p["shift1"])
        qkv = ref.int8_linear(h, p["wq_qkv"], p["ws_qkv"], p["b_qkv"]).reshape(rows, 3, HEADS, HEAD_DIM)
        ref.qk_norm_rope(qkv[:, 0], p["q_norm_w"], cos, sin)
        ref.qk_norm_rope(qkv[:, 1], p["k_norm_w"], cos, sin)
        a = ref.int8_linear(h, p["wq_out"], p["ws_out"], p["b_out"])
        y = ref.gate_residual(x, a, p["gate1"])
        h2 = ref.mod_scale_shift(ref.layer_norm_noaffine(y), p["scale2"], p["shift2"])
        f = ref.int8_linear(h2, p["wq_fc1"], p["ws_fc1"], p["b_fc1"])
        f = ref.int8_linear(f, p["wq_fc2"], p["ws_fc2"], p["b_fc2"], input_act="swiglu")
        return ref.gate_residual(y, f, p["gate2"])

    rowlocal()
    t0 = time.perf_counter()
    reps = 0
    while reps < 2 or time.perf_counter() - t0 < budget_s * 0.3:
        rowlocal()
        reps += 1
        if reps >= 20:
            break
    row_ms = (time.perf_counter() - t0) / reps * 1e3 * (tokens / rows)

    qrows = 128
    kf = torch.randn((tokens, HEAD_DIM), generator=g).to(torch.bfloat16)
    vf = torch.randn((tokens, HEAD_DIM), generator=g).to(torch.bfloat16)
    qf = torch.randn((qrows, HEAD_DIM), generator=g).to(torch.bfloat16)
    view = lambda t: t[None, None]
    ref.attention_rows_fp32(view(qf), view(kf), view(vf), 0, 0, qrows, HEAD_DIM ** -0.5)
    t0 = time.perf_counter()
    reps = 0
    while reps < 2 or time.perf_counter() - t0 < budget_s * 0.5:
        ref.attention_rows_fp32(view(qf), view(kf), view(vf), 0, 0, qrows, HEAD_DIM ** -0.5)
        reps += 1
        if reps >= 50:
            break
    attn_ms = (time.perf_counter() - t0) / reps * 1e3 * (tokens / qrows) * HEADS
    return {"value": row_ms + attn_ms, "unit": "ms", "cores": threads, "kind": "port",
            "sample": (f"row-local ops on {rows} of {tokens} rows (x{tokens / rows:.1f}); fp32 math attention "
                       f"for {qrows} query rows of 1 head vs all {tokens} keys (x{tokens / qrows:.1f} x {HEADS} heads); "
                       f"extrapolated; rowlocal {row_ms:.0f} ms + attention {attn_ms:.0f} ms"),
            "os_cpu_count": os.cpu_count()}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    vals = []
    per_step_budget = max(4.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    base = None
    for i in range(args.warmup + args.steps):
        base = cpu_block_ms(args.tokens, per_step_budget)
        if i >= args.warmup:
            vals.append(base["value"])
        if time.perf_counter() - t0 > 240 and len(vals) >= 1:
            break
    v = statistics.median(vals)
    base["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "ms", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": args.warmup, "ms_per_step": v, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8+bf16 (CPU: fp32 attention)",
            "data": "synthetic",
            "config": workload_config(args.tokens, 1, "cpu"),
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(tokens, world, par):
    return {"workload": f"one DiT block, {tokens} tokens, hidden {HIDDEN}, {HEADS}x{HEAD_DIM} heads, FFN {FFN} "
                        f"(BASELINE configs[3]/[4] structure)",
            "tokens": tokens, "hidden": HIDDEN, "heads": HEADS, "ffn": FFN, "parallelism": par,
            "l2": "inputs larger than L2 (activations >= 670 MB per step at 109099 tokens)"}


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------

def run_b200(args):
    import torch
    import torch.distributed as dist

    pkg = importlib.import_module("dcu-video-dit-turbo_b200")
    pkg._lib.load()   # raises when the CUDA library is missing: no fallback
    ops = pkg.ops
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    T = args.tokens
    sp = None
    splits = pkg.ulysses.sequence_splits(T, world)
    L = splits[rank]
    row0 = sum(splits[:rank])
    if world > 1:
        sp = pkg.ulysses.UlyssesSP(splits, HEADS, HEAD_DIM)
    local_heads = HEADS // world
    # auto: the most head chunks (all-to-all / attention overlap) whose attention launches
    # still fill their last wave of SMs
    chunks = args.head_chunks or (1 if world == 1 else pkg.ulysses.choose_head_chunks(T, local_heads))
    while local_heads % chunks:
        chunks -= 1
    params = pkg.block.make_block_params(HIDDEN, HEADS, HEAD_DIM, FFN, seed=0, device=dev)
    blk = pkg.block.DiTBlock(params, sp=sp, head_chunks=chunks, overlap=True,
                             fuse_residual=not args.no_fuse_residual)
    cos_all, sin_all = pkg.block.rope_tables(pkg.block.grid_positions(T))
    cos, sin = cos_all[row0:row0 + L].to(dev), sin_all[row0:row0 + L].to(dev)
    g = torch.Generator().manual_seed(1234 + rank)
    x_host = torch.randn((L, HIDDEN), generator=g).to(torch.bfloat16).pin_memory()
    out_host = torch.empty((L, HIDDEN), dtype=torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # attention kernel events (rank-local) recorded inside the timed steps
    attn_events = []
    orig_attn = blk._attn

    def timed_attn(q, k, v):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        o = orig_attn(q, k, v)
        e1.record()
        attn_events.append((e0, e1, q.shape[1], q.shape[2]))
        return o

    blk._attn = timed_attn

    for _ in range(args.warmup):
        y = blk.forward(x_dev, cos, sin)
    ops.check_device_status(dev)
    attn_events.clear()
    # single GPU: the pass is replayed from a CUDA graph (one launch instead of eleven);
    # the attention events are recorded inside the captured pass by a second, eager run
    use_graph = world == 1 and not args.no_graph
    run_step = lambda xin: blk.forward(xin, cos, sin)
    if use_graph:
        blk._attn = orig_attn
        graphed = pkg.block.GraphedBlock(blk, x_dev, cos, sin)
        run_step = lambda xin: graphed.replay()      # input already resident in the captured buffer

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    launches0 = ops.launch_count
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(args.steps):
        y = run_step(x_dev)
    end.record()
    barrier()
    launches = ops.launch_count - launches0
    ms_step = max_over_ranks(start.elapsed_time(end) / args.steps)
    if use_graph:
        # attention kernel time inside a long step: same pass, eager, with events around it
        blk._attn = timed_attn
        for _ in range(args.steps):
            blk.forward(x_dev, cos, sin)
        torch.cuda.synchronize()

    attn_ms = sum(e0.elapsed_time(e1) for e0, e1, _, _ in attn_events) / max(1, args.steps)
    attn_flops = sum(4.0 * s * s * h * HEAD_DIM for _, _, h, s in attn_events) / max(1, args.steps)
    attn_launches = len(attn_events) / max(1, args.steps)
    attn_ms = max_over_ranks(attn_ms)

    # end to end through the public API, as a serving loop would drive it: every step's
    # input shard comes from pinned host memory and every step's output goes back to pinned
    # host memory, inside the timed region.  Copies run on a side stream, double buffered,
    # so step i+1's upload and step i-1's download overlap step i's compute.
    blk._attn = orig_attn
    main = torch.cuda.current_stream(dev)
    side = torch.cuda.Stream(device=dev)
    x_bufs = [torch.empty_like(x_dev) for _ in range(2)]
    out_hosts = [out_host, torch.empty_like(out_host).pin_memory()]
    up_done = [torch.cuda.Event() for _ in range(2)]
    buf_free = [torch.cuda.Event() for _ in range(2)]
    for ev in buf_free:
        ev.record(main)

    def upload(i):
        with torch.cuda.stream(side):
            side.wait_event(buf_free[i % 2])          # the compute that read this buffer is done
            x_bufs[i % 2].copy_(x_host, non_blocking=True)
            up_done[i % 2].record(side)

    def e2e_loop(n):
        upload(0)
        pending = None
        for i in range(n):
            if i + 1 < n:
                upload(i + 1)
            main.wait_event(up_done[i % 2])
            # graph replays write one captured output buffer: clone it so that the download of
            # step i can overlap the replay of step i+1
            y = graphed(x_bufs[i % 2]).clone() if use_graph else blk.forward(x_bufs[i % 2], cos, sin)
            buf_free[i % 2].record(main)
            done = torch.cuda.Event()
            done.record(main)
            with torch.cuda.stream(side):
                side.wait_event(done)
                out_hosts[i % 2].copy_(y, non_blocking=True)
                y.record_stream(side)
            pending = y
        main.wait_stream(side)
        return pending

    e2e_loop(2)
    e2e_s, e2e_e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e2e_s.record()
    e2e_loop(args.steps)
    e2e_e.record()
    barrier()
    e2e_ms = max_over_ranks(e2e_s.elapsed_time(e2e_e) / args.steps)
    clocks = sampler.stop() if rank == 0 else None
    ops.check_device_status(dev)

    extra = {}
    if rank == 0 and world == 1 and T != 23638:
        # the 23638-token block (BASELINE configs[3]) in the same run, 1 GPU
        T2 = 23638
        c2, s2 = pkg.block.rope_tables(pkg.block.grid_positions(T2))
        c2, s2 = c2.to(dev), s2.to(dev)
        x2 = torch.randn((T2, HIDDEN), generator=g).to(torch.bfloat16).to(dev)
        blk1 = pkg.block.DiTBlock(params)
        for _ in range(3):
            blk1.forward(x2, c2, s2)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            blk1.forward(x2, c2, s2)
        b.record()
        torch.cuda.synchronize()
        extra["block_ms_23638_tokens"] = a.elapsed_time(b) / 10

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    pk = peaks()
    int8_ops = 2.0 * T * (HIDDEN * 3 * HIDDEN + HIDDEN * HIDDEN + HIDDEN * 2 * FFN + FFN * HIDDEN)
    # DRAM traffic of the attention kernel: 181.0 MB per launch measured with ncu at 8192 tokens x 24
    # heads (algorithmic 201 MB: q, k, v read and o written once; K/V re-reads come from L2), scaled
    # by the (token, head) rows this rank's launches cover
    attn_rows = sum(h * s for _, _, h, s in attn_events) / max(1, args.steps)
    attn_traffic = 181.0e6 / (8192 * 24) * attn_rows / max(1.0, attn_launches)
    roofline = {"kernel": "flash_fwd_kernel", "bound": "tensor",
                "achieved": attn_flops / (attn_ms * 1e-3) / 1e12 if attn_ms > 0 else None,
                "peak": pk["bf16_sustained"], "unit": "TFLOP/s",
                "peak_kind": f"dense bf16, sustained, {pk['source']}", "traffic": attn_traffic,
                "traffic_kind": "bytes per launch, scaled from the 8192-token ncu capture",
                "launches_per_step": attn_launches, "ms_per_step": attn_ms,
                "flops_per_step_per_gpu": attn_flops}
    roofline["frac"] = roofline["achieved"] / roofline["peak"] if roofline["achieved"] else None
    line = {"metric": METRIC, "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 GEMMs (s32 accumulate) + bf16 attention (f32 accumulate)",
            "data": "synthetic",
            "config": workload_config(T, world, f"ulysses_sp{world}_headchunks{chunks}" if world > 1
                                      else ("single_gpu_cuda_graph" if use_graph else "single_gpu")),
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
            "attn_tflops_per_gpu": roofline["achieved"],
            "int8_ops_per_step": int8_ops, **extra}
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_block_ms(T, args.cpu_seconds)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_kernel(args):
    """Kernel-only mode: device time of one kernel at the block's shape for `--tokens`
    rows, rotating over enough distinct buffers to exceed L2, against its roofline."""
    import torch

    pkg = importlib.import_module("dcu-video-dit-turbo_b200")
    ops = pkg.ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    T, pk = args.tokens, peaks()
    gen = torch.Generator(device=dev).manual_seed(7)
    rnd = lambda *shape: torch.randn(shape, device=dev, dtype=torch.float32, generator=gen).to(torch.bfloat16)
    ri8 = lambda *shape: torch.randint(-127, 128, shape, device=dev, dtype=torch.int8, generator=gen)
    vec = lambda n: (torch.randn((n,), device=dev, generator=gen) * 0.1).to(torch.bfloat16)

    def nbuf(bytes_each):
        return max(2, int(300e6 // max(1, bytes_each)) + 1)

    name = args.kernel
    if name == "flash":
        bufs = [rnd(T, 3, HEADS, HEAD_DIM) for _ in range(2)]
        views = [tuple(b[:, i].transpose(0, 1).unsqueeze(0) for i in range(3)) for b in bufs]
        fn = lambda i: ops.fwd_bhsd(*views[i % 2], HEAD_DIM ** -0.5)
        work, unit, peak, bound = 4.0 * T * T * HEADS * HEAD_DIM, "TFLOP/s", pk["bf16_burst"], "tensor"
    elif name in ("gemm_out_residual", "gemm_fc2_residual"):   # GEMM with the gated residual in its epilogue
        k, n = (HIDDEN, HIDDEN) if name == "gemm_out_residual" else (FFN, HIDDEN)
        a, w = ri8(T, k), ri8(n, k)
        rs, cs, b, gate = torch.rand(T, device=dev), torch.rand(n, device=dev) * 1e-4, vec(n), vec(n)
        xs = [rnd(T, n) for _ in range(nbuf(T * n * 2))]
        fn = lambda i: ops.int8_gemm_dequant_residual_(xs[i % len(xs)], gate, a, rs, w, cs, b)
        work, unit, peak, bound = 2.0 * T * n * k, "TOP/s", 2 * pk["bf16_burst"], "tensor"
    elif name.startswith("gemm"):
        k, n = {"gemm_qkv": (HIDDEN, 3 * HIDDEN), "gemm_fc1": (HIDDEN, 2 * FFN), "gemm_c1": (HIDDEN, HIDDEN),
                "gemm_fc2": (FFN, HIDDEN)}[name]
        a, w = ri8(T, k), ri8(n, k)
        rs, cs, b = torch.rand(T, device=dev), torch.rand(n, device=dev), vec(n)
        fn = lambda i: ops.int8_gemm_dequant(a, rs, w, cs, b)
        work, unit, peak, bound = 2.0 * T * n * k, "TOP/s", 2 * pk["bf16_burst"], "tensor"
    elif name == "quant":
        xs = [rnd(T, HIDDEN) for _ in range(nbuf(T * HIDDEN * 2))]
        fn = lambda i: ops.quantize_int8_rowwise(xs[i % len(xs)])
        work, unit, peak, bound = T * HIDDEN * 3 + T * 4, "GB/s", pk["hbm_gbs"], "hbm"
    elif name == "swiglu":
        xs = [rnd(T, 2 * FFN) for _ in range(nbuf(T * FFN * 4))]
        fn = lambda i: ops.swiglu_quantize_int8_rowwise(xs[i % len(xs)])
        work, unit, peak, bound = T * FFN * 5 + T * 4, "GB/s", pk["hbm_gbs"], "hbm"
    elif name in ("mod", "ln_quant", "gate"):
        xs = [rnd(T, HIDDEN) for _ in range(nbuf(T * HIDDEN * 2))]
        sc, sh = vec(HIDDEN), vec(HIDDEN)
        if name == "mod":
            fn = lambda i: ops.mod_scale_shift_(xs[i % len(xs)], sc, sh)
            work = T * HIDDEN * 4 + HIDDEN * 4
        elif name == "ln_quant":
            fn = lambda i: ops.layernorm_mod_quant(xs[i % len(xs)], sc, sh)
            work = T * HIDDEN * 3 + T * 4
        else:
            fn = lambda i: ops.gate_residual_(xs[i % len(xs)], xs[(i + 1) % len(xs)], sc)
            work = T * HIDDEN * 6
        unit, peak, bound = "GB/s", pk["hbm_gbs"], "hbm"
    elif name == "epilogue":
        n = 3 * HIDDEN
        accs = [torch.randint(-2000000, 2000000, (T, n), device=dev, dtype=torch.int32, generator=gen)
                for _ in range(nbuf(T * n * 4))]
        rs, cs = torch.rand(T, device=dev), torch.rand(n, device=dev)
        fn = lambda i: ops.epilogue_vec4(accs[i % len(accs)], rs, cs)
        work, unit, peak, bound = T * n * 6 + T * 4 + n * 4, "GB/s", pk["hbm_gbs"], "hbm"
    elif name == "frames_u8":   # 121 decoded frames 704x1280 RGB fp32 -> bytes (`--tokens` is ignored)
        n = 121 * 704 * 1280 * 3
        xs = [torch.rand((121, 704, 1280, 3), device=dev, generator=gen) for _ in range(2)]
        fn = lambda i: ops.images_to_u8(xs[i % 2])
        work, unit, peak, bound = n * 5, "GB/s", pk["hbm_gbs"], "hbm"
    elif name == "rope_pack":   # norm + rotary writing the all-to-all send buffer (8 ranks, 3 chunks)
        bufs = [rnd(T, 3, HEADS, HEAD_DIM) for _ in range(nbuf(T * 3 * HIDDEN * 2))]
        cos, sin = pkg.block.rope_tables(pkg.block.grid_positions(T))
        cos, sin, w = cos.to(dev), sin.to(dev), vec(HEAD_DIM) + 1
        fn = lambda i: ops.qk_norm_rope_pack(bufs[i % len(bufs)], w, w, cos, sin, 8, 3)
        work, unit, peak, bound = T * 3 * HIDDEN * 4 + T * 64 * 8, "GB/s", pk["hbm_gbs"], "hbm"
    elif name == "quant_gathered":   # quantizer reading the reverse all-to-all layout (8 ranks, 3 chunks)
        xs = [rnd(3, 8, T, HIDDEN // 24) for _ in range(nbuf(T * HIDDEN * 2))]
        fn = lambda i: ops.quantize_int8_rowwise_gathered(xs[i % len(xs)])
        work, unit, peak, bound = T * HIDDEN * 3 + T * 4, "GB/s", pk["hbm_gbs"], "hbm"
    else:  # rope
        bufs = [rnd(T, 3, HEADS, HEAD_DIM) for _ in range(nbuf(T * 3 * HIDDEN * 2))]
        cos, sin = pkg.block.rope_tables(pkg.block.grid_positions(T))
        cos, sin, w = cos.to(dev), sin.to(dev), vec(HEAD_DIM) + 1
        fn = lambda i: ops.qk_norm_rope_(bufs[i % len(bufs)], w, w, cos, sin)
        work, unit, peak, bound = T * 2 * HIDDEN * 4 + T * 64 * 8, "GB/s", pk["hbm_gbs"], "hbm"

    for i in range(args.warmup):
        fn(i)
    torch.cuda.synchronize()
    a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a_.record()
    for i in range(args.steps):
        fn(i)
    b_.record()
    torch.cuda.synchronize()
    ops.check_device_status(dev)
    ms = a_.elapsed_time(b_) / args.steps
    achieved = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    print(json.dumps({"kernel": name, "tokens": T, "ms": ms, "steps": args.steps, "warmup": args.warmup,
                      "roofline": {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                                   "frac": achieved / peak, "peak_kind": pk["source"] +
                                   (" (int8 = 2 x measured bf16 burst)" if unit == "TOP/s" else "")},
                      "algorithmic_work": work}))


def main():
    args = parse()
    if args.kernel:
        run_kernel(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
