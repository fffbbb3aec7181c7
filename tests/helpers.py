"""Input families shared by the parity tests (seeded, synthetic).

They follow the generators of the reference's own validators:
  kernels/exact-rowwise-int8/bench_exact_quantizer.py:35-88
  kernels/exact-rowwise-int8/validate_robustness.py:40-65
  kernels/swiglu-quant/bench_swiglu_quant.py:69-86
  kernels/int8-epilogue/bench.py:91-111
"""
import torch


def tile_pattern(values, m, k, dtype=torch.bfloat16):
    pattern = torch.tensor(values, dtype=torch.float32).to(dtype)
    count = m * k
    reps = (count + pattern.numel() - 1) // pattern.numel()
    return pattern.repeat(reps)[:count].reshape(m, k).contiguous()


def quantizer_families(m, k, seed=20260812):
    finfo = torch.finfo(torch.bfloat16)
    g = torch.Generator().manual_seed(seed + k)
    x = torch.randn((m, k), generator=g).to(torch.bfloat16)
    amps = torch.linspace(0.03125, 8.0, m, dtype=torch.float32)
    fams = {
        "random": (x * amps[:, None].to(torch.bfloat16)).contiguous(),
        "all_zero": torch.zeros((m, k), dtype=torch.bfloat16),
        "extreme_finite": tile_pattern([finfo.max, -finfo.max, finfo.tiny, -finfo.tiny, 1.0e-30,
                                        -1.0e-30, 0.0, -0.0, 1.0, -1.0], m, k),
        "round_even_boundaries": tile_pattern([127.0, -127.0, 126.5, 125.5, 2.5, 1.5, 0.5, -0.5,
                                               -1.5, -2.5, -125.5, -126.5, 0.0], m, k),
        "round_even_scale_0.5": tile_pattern([63.5, -63.5, 62.5, 1.25, 0.75, 0.25, -0.25, -0.75,
                                              -1.25, 0.0], m, k),
    }
    g2 = torch.Generator().manual_seed(seed + 1 + k)
    fams["random_plain"] = torch.randn((m, k), generator=g2).to(torch.bfloat16)
    nonfinite = fams["random_plain"].clone()
    if m >= 3 and k >= 6:
        nonfinite[0, :6] = torch.tensor([float("nan"), float("inf"), float("-inf"), 1.0, -1.0, 0.0]).to(torch.bfloat16)
        nonfinite[2, 1] = float("inf")
    fams["nan_and_infinities"] = nonfinite
    return fams


def swiglu_families(m, k, seed=20260812):
    finfo = torch.finfo(torch.bfloat16)
    g = torch.Generator().manual_seed(seed)
    return {
        "random": torch.randn((m, 2 * k), generator=g).to(torch.bfloat16),
        "zero": torch.zeros((m, 2 * k), dtype=torch.bfloat16),
        "extremes": tile_pattern([finfo.max, -finfo.max, finfo.tiny, -finfo.tiny, 0.0, -0.0, 127.0,
                                  -127.0, 2.5, -2.5, 1.5, -1.5, 0.5, -0.5], m, 2 * k),
    }


def epilogue_inputs(m, n, seed):
    g = torch.Generator().manual_seed(seed)
    acc = torch.randint(-2_000_000, 2_000_001, (m, n), dtype=torch.int32, generator=g)
    row = torch.rand((m,), generator=g) * 0.02 + 1e-5
    col = torch.rand((n,), generator=g) * 0.02 + 1e-5
    bias_bf16 = torch.randn((n,), generator=g).to(torch.bfloat16)
    bias_f32 = torch.randn((n,), generator=g)
    return acc, row, col, bias_bf16, bias_f32


def bits(t):
    """Bit-pattern view for exact comparison (NaN-safe)."""
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16)
    if t.dtype == torch.float32:
        return t.view(torch.int32)
    return t
