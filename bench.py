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

Timing follows the reference's protocol (kernels/exact-rowwise-int8/
bench_exact_quantizer.py:124-160 in the reference): warm-ups, then K rounds, each
between its own pair of CUDA events, worst rank per round, median over the rounds;
L2 is flushed between rounds.  Before anything is timed at N > 1 every rank runs the
single-GPU block on all T tokens and compares its own shard with the
sequence-parallel result (`sp_check`, as benchmarks/bench_sp_head_chunk_overlap.py:
264-323 does in the reference): a mismatch ends the run with exit code 2.

Prints ONE JSON line on rank 0.  `value` is the block time in ms, `e2e` the same
through the public API with the host->device copy of the input shard and the
device->host copy of the output inside the timed region.  `--impl reference` times
the CPU restatement of the reference's PyTorch path on a bounded sample of the same
workload on all host cores.
"""
from __future__ import annotations

import argparse
import importlib
import json
import math
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
SMALL_TOKENS = 23638           # the benchmark's second token count, timed in the same run
NVLINK_PEER_GBS = 770.0
INT8_NOMINAL_TOPS = 4500.0     # dense INT8, nominal; no measured INT8 peak exists on this pool
KERNEL_CHOICES = ["flash", "gemm_qkv", "gemm_fc1", "gemm_c1", "quant", "swiglu", "mod", "ln_quant",
                  "rope_pack", "quant_gathered", "gemm_out_residual", "gemm_fc2", "gemm_fc2_residual",
                  "frames_u8", "epilogue", "gate", "rope", "gemm_fc1_swiglu"]


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
    ap.add_argument("--no-fuse-swiglu", action="store_true",
                    help="fc1 and swiglu-quant as the reference's two operators instead of SwiGLU in fc1's epilogue")
    ap.add_argument("--no-graph", action="store_true", help="single GPU: launch the kernels one by one")
    ap.add_argument("--no-sp-check", action="store_true", help="skip the 1-GPU-vs-N-GPU parity gate")
    ap.add_argument("--exchange", default="peer", choices=["peer", "all_to_all"],
                    help="N > 1: how q/k/v and the attention output cross ranks: the kernels' own stores "
                         "into peer memory, or all-to-all collectives")
    ap.add_argument("--no-small", action="store_true", help=f"skip the {SMALL_TOKENS}-token leg")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel table (N=1)")
    ap.add_argument("--kernel", default=None, choices=KERNEL_CHOICES,
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

def host_threads() -> int:
    """All host cores for the CPU arm.  A launcher such as torchrun exports
    OMP_NUM_THREADS=1, which would otherwise leave the CPU arm on a single core."""
    import torch
    n = os.cpu_count() or 1
    torch.set_num_threads(n)
    return torch.get_num_threads()


class CpuSample:
    """The reference's PyTorch-CPU path on a bounded sample of one block, scaled to the block.

    Row-local ops (LayerNorm+modulation, quantizer, INT8 GEMM, epilogue, swiglu, RoPE,
    residual) run on a sample of `rows` token rows and scale by tokens/rows; attention runs
    one 2048-row query block of ONE head against ALL keys (the reference's sampled-block
    recipe, validation/validate_flash_longseq.py:62-71) and scales by
    (tokens/2048) x heads."""

    def __init__(self, tokens: int):
        import torch
        from oracle import ref_ops as ref

        self.ref, self.tokens, self.threads = ref, tokens, host_threads()
        g = torch.Generator().manual_seed(0)
        pkg = importlib.import_module("dcu-video-dit-turbo_b200")
        self.p = pkg.block.make_block_params(HIDDEN, HEADS, HEAD_DIM, FFN, seed=0, device="cpu")
        self.rows = min(2048, tokens)
        self.x = torch.randn((self.rows, HIDDEN), generator=g).to(torch.bfloat16)
        self.cos, self.sin = ref.rope_tables(pkg.block.grid_positions(self.rows))
        self.qrows = min(2048, tokens)
        view = lambda t: t[None, None]
        self.k = view(torch.randn((tokens, HEAD_DIM), generator=g).to(torch.bfloat16))
        self.v = view(torch.randn((tokens, HEAD_DIM), generator=g).to(torch.bfloat16))
        self.q = view(torch.randn((self.qrows, HEAD_DIM), generator=g).to(torch.bfloat16))
        self.rowlocal()
        self.attention()

    def rowlocal(self):
        ref, p, x, rows = self.ref, self.p, self.x, self.rows
        h = ref.mod_scale_shift(ref.layer_norm_noaffine(x), p["scale1"], p["shift1"])
        qkv = ref.int8_linear(h, p["wq_qkv"], p["ws_qkv"], p["b_qkv"]).reshape(rows, 3, HEADS, HEAD_DIM)
        ref.qk_norm_rope(qkv[:, 0], p["q_norm_w"], self.cos, self.sin)
        ref.qk_norm_rope(qkv[:, 1], p["k_norm_w"], self.cos, self.sin)
        a = ref.int8_linear(h, p["wq_out"], p["ws_out"], p["b_out"])
        y = ref.gate_residual(x, a, p["gate1"])
        h2 = ref.mod_scale_shift(ref.layer_norm_noaffine(y), p["scale2"], p["shift2"])
        f = ref.int8_linear(h2, p["wq_fc1"], p["ws_fc1"], p["b_fc1"])
        f = ref.int8_linear(f, p["wq_fc2"], p["ws_fc2"], p["b_fc2"], input_act="swiglu")
        return ref.gate_residual(y, f, p["gate2"])

    def attention(self):
        return self.ref.attention_rows_fp32(self.q, self.k, self.v, 0, 0, self.qrows, HEAD_DIM ** -0.5)

    @staticmethod
    def _time(fn, budget_s, max_reps):
        t0 = time.perf_counter()
        reps = 0
        while reps < 1 or (time.perf_counter() - t0 < budget_s and reps < max_reps):
            fn()
            reps += 1
        return (time.perf_counter() - t0) / reps

    def measure(self, budget_s: float) -> dict:
        tokens, rows, qrows = self.tokens, self.rows, self.qrows
        row_s = self._time(self.rowlocal, budget_s * 0.3, 20)
        attn_s = self._time(self.attention, budget_s * 0.6, 50)
        row_ms = row_s * 1e3 * (tokens / rows)
        attn_ms = attn_s * 1e3 * (tokens / qrows) * HEADS
        return {"value": row_ms + attn_ms, "unit": "ms", "cores": self.threads, "kind": "port",
                "extrapolated": True,
                "sample": (f"row-local ops on {rows} of {tokens} rows ({row_s * 1e3:.0f} ms measured, "
                           f"x{tokens / rows:.1f}); fp32 math attention for one {qrows}-row query block of 1 head "
                           f"vs all {tokens} keys ({attn_s * 1e3:.0f} ms measured, x{tokens / qrows:.1f} blocks x "
                           f"{HEADS} heads); extrapolated total: rowlocal {row_ms:.0f} ms + attention {attn_ms:.0f} ms"),
                "os_cpu_count": os.cpu_count()}


def cpu_block_ms(tokens: int, budget_s: float) -> dict:
    return CpuSample(tokens).measure(budget_s)


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    t0 = time.perf_counter()
    vals = []
    per_step_budget = max(2.0, min(20.0, 100.0 / max(1, args.steps + args.warmup)))
    base = None
    sample = CpuSample(args.tokens)
    for i in range(args.warmup + args.steps):
        base = sample.measure(per_step_budget)
        if i >= args.warmup:
            vals.append(base["value"])
        if time.perf_counter() - t0 > 200 and len(vals) >= 1:
            break
    v = statistics.median(vals)
    base["value"] = v
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": "ms", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": args.warmup, "ms_per_step": v, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8+bf16 (CPU: fp32 attention)",
            "data": "synthetic",
            "config": workload_config(args.tokens),
            "parallelism": f"cpu_{base['cores']}_threads",
            "cpu_baseline": base,
            "e2e": {"value": v, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(tokens):
    """Names the workload only (identical for both arms)."""
    return {"workload": f"one DiT block, {tokens} tokens, hidden {HIDDEN}, {HEADS}x{HEAD_DIM} heads, FFN {FFN}",
            "tokens": tokens, "hidden": HIDDEN, "heads": HEADS, "ffn": FFN,
            "l2": "L2 flushed between timed rounds; activations >= 670 MB per step at 109099 tokens"}


# --------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------

class Job:
    """One rank's view of the block at a token count: shard bounds, block, rotary tables."""

    def __init__(self, pkg, params, tokens, world, rank, dev, head_chunks, fuse_residual, exchange="all_to_all",
                 fuse_swiglu=True):
        self.pkg, self.tokens, self.world, self.rank, self.dev = pkg, tokens, world, rank, dev
        self.exchange, self.exchange_note = ("all_to_all" if world > 1 else None), None
        self.splits = pkg.ulysses.sequence_splits(tokens, world)
        self.L = self.splits[rank]
        self.row0 = sum(self.splits[:rank])
        self.sp = pkg.ulysses.UlyssesSP(self.splits, HEADS, HEAD_DIM) if world > 1 else None
        local_heads = HEADS // world
        # auto: the most head chunks (all-to-all / attention overlap) whose attention launches
        # still fill their last wave of SMs
        chunks = head_chunks or (1 if world == 1 else pkg.ulysses.choose_head_chunks(tokens, local_heads))
        while local_heads % chunks:
            chunks -= 1
        if world > 1 and exchange == "peer":
            # collective: succeeds or raises on every rank alike
            try:
                self.sp.enable_peer_exchange(dev)
                self.exchange, chunks = "peer", 1
            except RuntimeError as exc:
                self.exchange_note = f"peer exchange unavailable, using all-to-all collectives: {exc}"
        self.chunks = chunks
        self.params = params
        self.block = pkg.block.DiTBlock(params, sp=self.sp, head_chunks=chunks, overlap=True,
                                        fuse_residual=fuse_residual, fuse_swiglu=fuse_swiglu)
        cos_all, sin_all = pkg.block.rope_tables(pkg.block.grid_positions(tokens))
        self.cos_all, self.sin_all = cos_all.to(dev), sin_all.to(dev)
        self.cos = self.cos_all[self.row0:self.row0 + self.L].contiguous()
        self.sin = self.sin_all[self.row0:self.row0 + self.L].contiguous()

    def full_input(self, seed):
        """All T rows, identical on every rank (same device generator seed)."""
        import torch
        g = torch.Generator(device=self.dev).manual_seed(seed)
        return torch.randn((self.tokens, HIDDEN), device=self.dev, dtype=torch.float32,
                           generator=g).to(torch.bfloat16)

    def shard(self, full):
        return full[self.row0:self.row0 + self.L].contiguous()

    def parallelism(self):
        if self.world == 1:
            return None
        how = "peer_stores" if self.exchange == "peer" else f"all_to_all_headchunks{self.chunks}"
        return f"ulysses_sp{self.world}_{how}"

    def close(self):
        if self.sp is not None and self.sp.peer is not None:
            self.sp.peer.close()
            self.sp.peer = None


def sp_check(job: Job, dist) -> dict:
    """Parity gate inside the distributed run: the single-GPU block on ALL tokens, computed
    locally by every rank, against this rank's shard of the sequence-parallel block
    (bitwise and PSNR), and the sequence-parallel attention rows against fp32 math
    attention on the reference's sampled heads and row blocks
    (validation/validate_flash_longseq.py:62-71 in the reference)."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = False
    pkg, dev, T = job.pkg, job.dev, job.tokens
    x_full = job.full_input(4321)
    taps1, taps2 = {}, {}
    single = pkg.block.DiTBlock(job.params, fuse_residual=job.block.fuse_residual,
                                fuse_swiglu=job.block.fuse_swiglu)
    y1 = single.forward(x_full, job.cos_all, job.sin_all, taps=taps1)
    y2 = job.block.forward(job.shard(x_full), job.cos, job.sin, taps=taps2)
    torch.cuda.synchronize()
    sl = slice(job.row0, job.row0 + job.L)
    want = y1[sl]
    block_equal = bool(torch.equal(y2, want))
    attn_equal = bool(torch.equal(taps2["attn"], taps1["attn"][sl]))
    mse = float(((want.double() - y2.double()) ** 2).mean())
    peak = float(want.float().max() - want.float().min())
    psnr = float("inf") if mse == 0.0 else 10.0 * math.log10(peak * peak / mse)
    # sampled rows of the sequence-parallel attention output vs fp32 math attention
    qkv = taps1["qkv"]
    got_all = taps2["attn"].view(job.L, HEADS, HEAD_DIM)
    err, ref_max, rows_checked = 0.0, 0.0, 0
    scale = HEAD_DIM ** -0.5
    for head in (0, HEADS // 2, HEADS - 1):
        kf, vf = qkv[:, 1, head].float(), qkv[:, 2, head].float()
        for r0 in (0, T // 2, max(0, T - 2048)):
            a, b = max(r0, job.row0), min(min(T, r0 + 2048), job.row0 + job.L)
            if a >= b:
                continue
            ref = torch.softmax((qkv[a:b, 0, head].float() @ kf.T) * scale, dim=-1) @ vf
            got = got_all[a - job.row0:b - job.row0, head].float()
            err = max(err, float((got - ref).abs().max()))
            ref_max = max(ref_max, float(ref.abs().max()))
            rows_checked += b - a
    stats = torch.tensor([float(block_equal), float(attn_equal), min(psnr, 1e9), -err, -ref_max],
                         device=dev, dtype=torch.float64)
    dist.all_reduce(stats, op=dist.ReduceOp.MIN)
    rows_t = torch.tensor([rows_checked], device=dev, dtype=torch.int64)
    dist.all_reduce(rows_t, op=dist.ReduceOp.SUM)
    err, ref_max = -float(stats[3]), -float(stats[4])
    tol = max(2e-4, 2.0 ** -7 * ref_max)
    out = {"tokens": T, "world": job.world, "head_chunks": job.chunks, "exchange": job.exchange,
           "bitwise_equal": bool(stats[0] == 1.0), "attention_rows_bitwise_equal": bool(stats[1] == 1.0),
           "psnr_db": None if float(stats[2]) >= 1e9 else float(stats[2]),
           "psnr_note": "null = infinite (no differing element on any rank)",
           "attn_max_abs_err_sampled_rows": err, "attn_tolerance": tol,
           "attn_rows_checked": int(rows_t.item()),
           "attn_reference": "fp32 math attention on the device (TF32 off), heads {0,12,23} x row blocks "
                             "{0, T/2, T-2048} of 2048 rows"}
    out["passed"] = bool(out["bitwise_equal"] and out["attention_rows_bitwise_equal"] and err <= tol
                         and (out["psnr_db"] is None or out["psnr_db"] >= 60.0))
    del taps1, taps2, y1, y2, x_full, qkv
    torch.cuda.empty_cache()
    return out


class Timing:
    """Rounds of one step each between their own CUDA events, L2 flushed between rounds,
    worst rank per round, median over rounds."""

    def __init__(self, dev, world, dist):
        import torch
        self.torch, self.dev, self.world, self.dist = torch, dev, world, dist
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)   # 2 x L2

    def barrier(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, values):
        t = self.torch.tensor(values, device=self.dev, dtype=self.torch.float64)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    def rounds(self, step, n):
        torch = self.torch
        events = []
        self.barrier()
        for _ in range(n):
            self.flush_buf.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            step()
            e1.record()
            events.append((e0, e1))
        self.barrier()
        per_round = self.max_over_ranks([a.elapsed_time(b) for a, b in events])
        return {"median": statistics.median(per_round), "mean": sum(per_round) / len(per_round),
                "min": min(per_round), "max": max(per_round), "rounds": len(per_round)}


def kernel_table(pkg, block, x, cos, sin, pk, passes=3):
    """One eager pass of the block with CUDA events around every launch: per kernel its
    time, achieved rate and fraction of the roofline that bounds it."""
    ops = pkg.ops
    block.forward(x, cos, sin)
    with ops.LaunchTimer() as timer:
        for _ in range(passes):
            block.forward(x, cos, sin)
    recs = timer.results()
    per = len(recs) // passes
    labels = ["layernorm_mod_quant (adaLN 1)", "int8_gemm_dequant qkv 3072->9216", "qk_norm_rope",
              "flash_fwd", "quantize_int8_rowwise (attention rows)",
              "int8_gemm_dequant_residual out 3072->3072", "layernorm_mod_quant (adaLN 2)",
              "int8_gemm_dequant fc1 3072->16384", "swiglu_quantize_int8_rowwise",
              "int8_gemm_dequant_residual fc2 8192->3072"]
    if getattr(block, "fuse_swiglu", False):
        labels[7:9] = ["int8_gemm_dequant_swiglu fc1 3072->16384 (SwiGLU in the epilogue)",
                       "quantize_int8_rowwise (SwiGLU product, 8192 wide)"]
    rows = []
    for i in range(per):
        ms = statistics.median(recs[p * per + i]["ms"] for p in range(passes))
        rec = recs[i]
        rows.append(kernel_row(labels[i] if per == len(labels) else rec["name"], rec["name"], ms,
                               rec["bound"], rec["work"], pk))
    return rows


def kernel_row(label, entry, ms, bound, work, pk):
    row = {"kernel": label, "entry": entry, "ms": ms, "bound": bound, "work": work}
    if bound == "hbm":
        row.update(unit="GB/s", achieved=work / ms / 1e6, peak=pk["hbm_gbs"], peak_kind=f"HBM copy, {pk['source']}")
    elif bound == "int8":
        row.update(unit="TOP/s", achieved=work / ms / 1e9, peak=2 * pk["bf16_burst"],
                   peak_kind=f"ASSUMED 2 x bf16 burst ({pk['source']}); no measured INT8 peak",
                   frac_of_nominal_4500=work / ms / 1e9 / INT8_NOMINAL_TOPS)
    elif bound == "bf16":
        row.update(unit="TFLOP/s", achieved=work / ms / 1e9, peak=pk["bf16_sustained"],
                   peak_kind=f"dense bf16 sustained, {pk['source']}")
    elif bound == "nvlink":
        # bytes this GPU stores into its peers' memory; 770 GB/s is the peer-copy rate per
        # direction measured on this pool's B200s (nominal 900)
        row.update(unit="GB/s", achieved=work / ms / 1e6, peak=NVLINK_PEER_GBS,
                   peak_kind="NVLink peer copy per direction, measured on this pool (nominal 900)")
    if "achieved" in row:
        row["frac"] = row["achieved"] / row["peak"]
    return row


def standalone_rows(pkg, tokens, dev, pk):
    """The memory-bound operators timed ALONE on rotating buffers larger than L2: the two that
    the block only runs fused (mod-scale-shift inside LayerNorm, the quantizer of a plain bf16
    tensor), and the two producer fusions (LayerNorm + modulation + quantizer, swiglu-quant),
    whose in-block rows above are taken right after attention has pulled the SM clock down
    under the power cap (both are instruction-issue-bound, so they follow the clock)."""
    import torch
    ops = pkg.ops
    g = torch.Generator(device=dev).manual_seed(3)
    n_buf = max(2, int(300e6 // (tokens * HIDDEN * 2)) + 1)
    xs = [torch.randn((tokens, HIDDEN), device=dev, generator=g).to(torch.bfloat16) for _ in range(n_buf)]
    sc = (torch.randn((HIDDEN,), device=dev, generator=g) * 0.1).to(torch.bfloat16)
    sh = (torch.randn((HIDDEN,), device=dev, generator=g) * 0.1).to(torch.bfloat16)
    rows = []

    def timed(label, shape, fn):
        for i in range(3):
            fn(i)
        with ops.LaunchTimer() as timer:
            for i in range(11):
                fn(i)
        recs = timer.results()
        rows.append(kernel_row(f"{label} {shape}", recs[0]["name"],
                               statistics.median(r["ms"] for r in recs), recs[0]["bound"], recs[0]["work"], pk))

    timed("mod_scale_shift (standalone)", f"{tokens}x{HIDDEN}", lambda i: ops.mod_scale_shift_(xs[i % n_buf], sc, sh))
    timed("quantize_int8_rowwise (standalone)", f"{tokens}x{HIDDEN}", lambda i: ops.quantize_int8_rowwise(xs[i % n_buf]))
    timed("layernorm_mod_quant (standalone)", f"{tokens}x{HIDDEN}",
          lambda i: ops.layernorm_mod_quant(xs[i % n_buf], sc, sh))
    del xs
    torch.cuda.empty_cache()
    wide = [torch.randn((tokens, 2 * FFN), device=dev, generator=g).to(torch.bfloat16) for _ in range(2)]
    timed("swiglu_quantize_int8_rowwise (standalone)", f"{tokens}x{2 * FFN}",
          lambda i: ops.swiglu_quantize_int8_rowwise(wide[i % 2]))
    del wide
    torch.cuda.empty_cache()
    return rows


def checked_job(pkg, params, tokens, world, rank, dev, args, dist, checks):
    """A Job at `tokens` that has passed the parity gate (N > 1), or exit 2.  If the peer
    exchange fails the gate, that is recorded in `exchange_note` (and in the failed check kept
    beside it) and the job is rebuilt on all-to-all collectives, which must then pass."""
    job = Job(pkg, params, tokens, world, rank, dev, args.head_chunks, not args.no_fuse_residual, args.exchange,
              not args.no_fuse_swiglu)
    if world == 1 or args.no_sp_check:
        return job
    check = sp_check(job, dist)
    pkg.ops.check_device_status(dev)
    if not check["passed"] and job.exchange == "peer":
        failed = check
        job.close()
        job = Job(pkg, params, tokens, world, rank, dev, args.head_chunks, not args.no_fuse_residual, "all_to_all",
                  not args.no_fuse_swiglu)
        job.exchange_note = "the peer exchange FAILED the parity gate; timed with all-to-all collectives instead"
        check = sp_check(job, dist)
        check["failed_peer_check"] = failed
    checks.append(check)
    if not check["passed"]:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "n_gpus": world, "error": "sequence-parallel output differs "
                              "from the single-GPU block", "sp_check": check}))
        dist.destroy_process_group()
        sys.exit(2)
    return job


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
    params = pkg.block.make_block_params(HIDDEN, HEADS, HEAD_DIM, FFN, seed=0, device=dev)
    # ---- parity gate inside the distributed run (before anything is timed) ----
    checks = []
    job = checked_job(pkg, params, T, world, rank, dev, args, dist, checks)
    blk, cos, sin, L = job.block, job.cos, job.sin, job.L
    timing = Timing(dev, world, dist)

    x_dev = job.shard(job.full_input(1234))
    x_host = x_dev.cpu().pin_memory()
    out_host = torch.empty((L, HIDDEN), dtype=torch.bfloat16).pin_memory()

    # attention kernel events (rank-local) recorded inside timed steps
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
    # single GPU: the pass is replayed from a CUDA graph (one launch instead of ten); the
    # attention events are then recorded by a second, eager run of the same steps
    use_graph = world == 1 and not args.no_graph
    run_step = lambda: blk.forward(x_dev, cos, sin)
    if use_graph:
        blk._attn = orig_attn
        graphed = pkg.block.GraphedBlock(blk, x_dev, cos, sin)
        run_step = graphed.replay      # input already resident in the captured buffer

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ops.launch_count
    main_timing = timing.rounds(run_step, args.steps)
    launches = ops.launch_count - launches0
    ms_step = main_timing["median"]
    if use_graph:
        blk._attn = timed_attn
        for _ in range(args.steps):
            timing.flush_buf.zero_()
            blk.forward(x_dev, cos, sin)
        torch.cuda.synchronize()

    steps_seen = max(1, args.steps)
    attn_ms = timing.max_over_ranks([sum(e0.elapsed_time(e1) for e0, e1, _, _ in attn_events) / steps_seen])[0]
    attn_flops = sum(4.0 * s * s * h * HEAD_DIM for _, _, h, s in attn_events) / steps_seen
    attn_launches = len(attn_events) / steps_seen
    attn_rows = sum(h * s for _, _, h, s in attn_events) / steps_seen

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
        main.wait_stream(side)

    def e2e_serial_step():
        """Latency form: upload, block, download, one after the other on one stream."""
        x_bufs[0].copy_(x_host, non_blocking=True)
        y = graphed(x_bufs[0]) if use_graph else blk.forward(x_bufs[0], cos, sin)
        out_hosts[0].copy_(y, non_blocking=True)

    e2e_loop(2)
    e2e_s, e2e_e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    timing.barrier()
    e2e_s.record()
    e2e_loop(args.steps)
    e2e_e.record()
    timing.barrier()
    e2e_ms = timing.max_over_ranks([e2e_s.elapsed_time(e2e_e) / args.steps])[0]
    e2e_serial_step()
    e2e_latency = timing.rounds(e2e_serial_step, min(5, args.steps))
    clocks = sampler.stop() if rank == 0 else None
    ops.check_device_status(dev)

    pk = peaks()
    # per-kernel table: every rank runs the passes (they contain collectives), rank 0 reports.
    # At N > 1 the rows are this rank's kernels; what the step takes beyond their sum is the
    # exposed part of the all-to-alls plus launch gaps.
    kernels = None
    if not args.no_kernels:
        kernels = kernel_table(pkg, blk, x_dev, cos, sin, pk)
        if world == 1:
            kernels += standalone_rows(pkg, T, dev, pk)

    # ---- the second token count of the metric (23638), same ranks, same protocol ----
    small = None
    if T != SMALL_TOKENS and not args.no_small:
        torch.cuda.empty_cache()
        job2 = checked_job(pkg, params, SMALL_TOKENS, world, rank, dev, args, dist, checks)
        x2 = job2.shard(job2.full_input(1235))
        step2 = lambda: job2.block.forward(x2, job2.cos, job2.sin)
        for _ in range(max(3, args.warmup)):
            step2()
        if world == 1 and not args.no_graph:
            step2 = pkg.block.GraphedBlock(job2.block, x2, job2.cos, job2.sin).replay
        t2 = timing.rounds(step2, max(11, args.steps))
        small = {"tokens": SMALL_TOKENS, "ms": t2["median"], "timing": t2, "head_chunks": job2.chunks,
                 "parallelism": (job2.parallelism() if world > 1 else
                                 ("single_gpu_cuda_graph" if not args.no_graph else "single_gpu"))}
        if job2.exchange_note:
            small["exchange_note"] = job2.exchange_note
        if kernels is not None:
            small["kernels"] = kernel_table(pkg, job2.block, x2, job2.cos, job2.sin, pk, passes=5)
            small["kernels_ms_sum"] = sum(k["ms"] for k in small["kernels"])
            if world == 1:
                small["kernels"] += standalone_rows(pkg, SMALL_TOKENS, dev, pk)
        ops.check_device_status(dev)

    if small is not None:
        job2.close()
    job.close()
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    int8_ops = 2.0 * T * (HIDDEN * 3 * HIDDEN + HIDDEN * HIDDEN + HIDDEN * 2 * FFN + FFN * HIDDEN)
    # DRAM traffic of the attention kernel: 181.0 MB per launch measured with ncu at 8192 tokens x 24
    # heads (algorithmic 201 MB: q, k, v read and o written once; K/V re-reads come from L2), scaled
    # by the (token, head) rows this rank's launches cover
    attn_traffic = 181.0e6 / (8192 * 24) * attn_rows / max(1.0, attn_launches)
    roofline = {"kernel": "flash_fwd_kernel", "bound": "tensor",
                "achieved": attn_flops / (attn_ms * 1e-3) / 1e12 if attn_ms > 0 else None,
                "peak": pk["bf16_sustained"], "unit": "TFLOP/s",
                "peak_kind": f"dense bf16, sustained, {pk['source']}", "traffic": attn_traffic,
                "traffic_kind": "bytes per launch, scaled from the 8192-token ncu capture",
                "launches_per_step": attn_launches, "ms_per_step": attn_ms,
                "flops_per_step_per_gpu": attn_flops,
                "timed_in": ("a second, eager pass of the same steps after the graph-timed rounds "
                             "(CUDA events around the launch)" if use_graph else
                             "the timed rounds (CUDA events around each launch)")}
    roofline["frac"] = roofline["achieved"] / roofline["peak"] if roofline["achieved"] else None
    if clocks and clocks.get("sm_mhz") and roofline["achieved"]:
        # clock-normalised: fraction of what the tensor pipe can do at the sampled SM clock
        roofline["frac_of_pipe_at_sampled_clock"] = (
            roofline["achieved"] * 1e12 / (8192.0 * 148 * clocks["sm_mhz"] * 1e6))
    par = job.parallelism() if world > 1 else ("single_gpu_cuda_graph" if use_graph else "single_gpu")
    line = {"metric": METRIC, "value": ms_step, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "int8 GEMMs (s32 accumulate) + bf16 attention (f32 accumulate)",
            "data": "synthetic",
            "config": workload_config(T),
            "parallelism": par,
            "timing": dict(main_timing, protocol="one step per round between its own CUDA events, L2 flushed "
                                                 "between rounds, worst rank per round, median over rounds"),
            "e2e": {"value": e2e_ms, "unit": "ms", "kind": "pipelined", "h2d_bytes_per_step": x_host.numel() * 2,
                    "d2h_bytes_per_step": out_host.numel() * 2,
                    "note": "throughput form: copies double-buffered on a side stream overlap the next step",
                    "latency_ms": e2e_latency["median"],
                    "latency_note": "serial form: upload, block, download on one stream, median of rounds"},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
            "attn_tflops_per_gpu": roofline["achieved"],
            "int8_ops_per_step": int8_ops}
    if job.exchange_note:
        line["exchange_note"] = job.exchange_note
    if checks:
        line["sp_check"] = checks[0]
        if len(checks) > 1:
            line["sp_check_23638"] = checks[1]
    if small is not None:
        line["block_ms_23638_tokens"] = small["ms"]
        line["block_23638"] = small
    if kernels is not None:
        line["kernels"] = kernels
        line["kernels_ms_sum"] = sum(k["ms"] for k in kernels if "standalone" not in k["kernel"])
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_block_ms(T, args.cpu_seconds)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_kernel(args):
    """Kernel-only mode: device time of one kernel at the block's shape for `--tokens`
    rows, rotating over enough distinct buffers to exceed L2, against its roofline.
    11 rounds of `--steps` calls, median (the reference's protocol)."""
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
    elif name == "gemm_fc1_swiglu":   # first FFN projection with SwiGLU in the epilogue (values random: timing only)
        k, n = HIDDEN, 2 * FFN
        a, w = ri8(T, k), ri8(n, k)
        rs, cs, b = torch.rand(T, device=dev) * 1e-2, torch.rand(n, device=dev) * 1e-2, vec(n)
        fn = lambda i: ops.int8_gemm_dequant_swiglu(a, rs, w, cs, b)
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

    for i in range(max(3, args.warmup)):
        fn(i)
    torch.cuda.synchronize()
    n_rounds = 1 if name == "flash" and T > 50000 else 11
    per_round = []
    call = 0
    for _ in range(n_rounds):
        a_, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_.record()
        for _ in range(args.steps):
            fn(call)
            call += 1
        b_.record()
        torch.cuda.synchronize()
        per_round.append(a_.elapsed_time(b_) / args.steps)
    ops.check_device_status(dev)
    ms = statistics.median(per_round)
    achieved = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    roofline = {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                "peak_kind": pk["source"] + (" (ASSUMED: int8 = 2 x measured bf16 burst; no measured INT8 peak)"
                                             if unit == "TOP/s" else "")}
    if unit == "TOP/s":
        roofline["frac_of_nominal_4500"] = achieved / INT8_NOMINAL_TOPS
    print(json.dumps({"kernel": name, "tokens": T, "ms": ms, "ms_min": min(per_round), "ms_max": max(per_round),
                      "rounds": n_rounds, "calls_per_round": args.steps, "warmup": max(3, args.warmup),
                      "roofline": roofline, "algorithmic_work": work}))


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
