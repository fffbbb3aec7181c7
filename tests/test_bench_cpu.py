"""bench.py without a GPU: the reference arm's JSON line (the oracle's CPU path on a bounded
sample, all host cores), the roofline arithmetic of a per-kernel row, and the workload
description shared by both arms."""
import importlib.util
import json
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_reference_arm_line_on_a_small_token_count():
    env = dict(os.environ, OMP_NUM_THREADS="1")      # what a multi-process launcher exports
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--tokens", "512",
                          "--steps", "1", "--warmup", "0"], capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["metric"] == "dit_block_ms" and line["unit"] == "ms"
    assert line["higher_is_better"] is False and line["value"] > 0
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["extrapolated"] is True and "sample" in base
    # every host core is used even though the environment asked for one thread
    assert base["cores"] == os.cpu_count()
    assert line["e2e"] == {"value": line["value"], "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    # the workload description is the same object the GPU arm prints: no arm-specific key in it
    assert line["config"] == _bench().workload_config(512) and "parallelism" not in line["config"]


def test_other_ranks_of_the_reference_arm_do_nothing():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--tokens", "512",
                          "--steps", "1", "--warmup", "0", "--gpus", "2"], capture_output=True, text=True,
                         timeout=120, env=env)
    assert out.returncode == 0 and out.stdout.strip() == ""


def test_kernel_row_rates():
    b = _bench()
    pk = {"hbm_gbs": 6000.0, "bf16_burst": 1700.0, "bf16_sustained": 1400.0, "source": "measured"}
    hbm = b.kernel_row("k", "b2_k", 2.0, "hbm", 6_000_000_000, pk)           # 6 GB in 2 ms = 3000 GB/s
    assert abs(hbm["achieved"] - 3000.0) < 1e-6 and abs(hbm["frac"] - 0.5) < 1e-9 and hbm["unit"] == "GB/s"
    i8 = b.kernel_row("g", "b2_g", 1.0, "int8", 1_700_000_000_000, pk)       # 1.7e12 ops in 1 ms = 1700 TOP/s
    assert abs(i8["achieved"] - 1700.0) < 1e-6 and abs(i8["frac"] - 0.5) < 1e-9
    assert "ASSUMED" in i8["peak_kind"] and abs(i8["frac_of_nominal_4500"] - 1700.0 / 4500.0) < 1e-9
    bf = b.kernel_row("f", "b2_f", 10.0, "bf16", 7_000_000_000_000, pk)      # 7e12 flop in 10 ms = 700 TFLOP/s
    assert abs(bf["achieved"] - 700.0) < 1e-6 and abs(bf["frac"] - 0.5) < 1e-9
    assert "achieved" not in b.kernel_row("x", "b2_x", 1.0, None, None, pk)
    # kernels that store into peer GPUs are accounted against the measured peer-copy rate
    nv = b.kernel_row("s", "b2_s", 0.1, "nvlink", 38_500_000, pk)            # 38.5 MB in 0.1 ms = 385 GB/s
    assert nv["unit"] == "GB/s" and abs(nv["achieved"] - 385.0) < 1e-6 and abs(nv["frac"] - 0.5) < 1e-9
    assert nv["peak"] == b.NVLINK_PEER_GBS


def test_exchange_and_fusion_flags_parse():
    b = _bench()
    old = sys.argv
    try:
        sys.argv = ["bench.py"]
        args = b.parse()
        assert args.exchange == "peer" and not args.no_fuse_swiglu and not args.no_fuse_residual
        sys.argv = ["bench.py", "--exchange", "all_to_all", "--no-fuse-swiglu", "--kernel", "gemm_fc1_swiglu"]
        args = b.parse()
        assert args.exchange == "all_to_all" and args.no_fuse_swiglu and args.kernel == "gemm_fc1_swiglu"
    finally:
        sys.argv = old
