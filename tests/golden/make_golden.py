"""Generate the golden fixtures in this directory FROM THE REFERENCE'S OWN PYTHON.

Run once where the reference checkout is available (REFERENCE_ROOT=<path to it>
python make_golden.py); the fixtures are committed, this script documents how they were
made and can regenerate them.  Nothing else reads the reference tree.

What is extracted (by `ast`, the way the reference's own contract verifier does in
kernels/int8-epilogue-vec4/verify_v11_contract.py:42-61, because the files load
device DSOs at import time and cannot be imported whole):
  * eager_epilogue           kernels/int8-epilogue/bench.py:33-48
  * _vec4_epilogue_gate      launcher/benchmark_launcher_v14_hires_int8_candidate.py:863-904
  * _exact_quantizer_gate    launcher/benchmark_launcher_v14_hires_int8_candidate.py:157-179
  * ref_rows                 validation/validate_flash_longseq.py:37-42
  * exact_fp32               benchmarks/bench_opendas_h3_flash_bshd.py:71-74
and run on seeded CPU inputs.  The quantizer known-answer vectors are hand-derived
from the reference's comments (kernels/exact-rowwise-int8/bench_exact_quantizer.py:63-84,
validate_robustness.py:48-65, quantizer_kernel.hip:68-73,101-104) and written by
this script as well.
"""
from __future__ import annotations

import ast
import json
import os
import struct
from pathlib import Path

import numpy as np
import torch

REF = Path(os.environ["REFERENCE_ROOT"])   # path of the reference checkout
OUT = Path(__file__).resolve().parent


def extract(path: Path, names: set[str], namespace: dict) -> dict:
    tree = ast.parse(path.read_text())
    fns = [n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name in names]
    assert {f.name for f in fns} == names, (path, names)
    exec(compile(ast.Module(body=fns, type_ignores=[]), str(path), "exec"), namespace)
    return namespace


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().astype(np.uint16)


def f32bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


class FakeTensor:
    def __init__(self, shape, dtype, *, contiguous=True, device="cuda:0", is_cuda=True,
                 requires_grad=False):
        self.shape = shape
        self.dtype = dtype
        self.is_cuda = is_cuda
        self.device = device
        self.requires_grad = requires_grad
        self._contiguous = contiguous

    def is_contiguous(self):
        return self._contiguous

    def dim(self):
        return len(self.shape)

    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n


def golden_epilogue():
    ns = extract(REF / "kernels/int8-epilogue/bench.py", {"eager_epilogue"}, {"torch": torch})
    eager = ns["eager_epilogue"]
    out = {}
    for idx, (m, n, seed) in enumerate(((37, 52, 20260810), (64, 256, 20260811), (5, 7, 20260812))):
        g = torch.Generator().manual_seed(seed)
        acc = torch.randint(-2_000_000, 2_000_001, (m, n), dtype=torch.int32, generator=g)
        row = torch.rand((m, 1), generator=g) * 0.02 + 1e-5
        col = torch.rand((n,), generator=g) * 0.02 + 1e-5
        bias_bf16 = torch.randn((n,), generator=g).to(torch.bfloat16)
        bias_f32 = torch.randn((n,), generator=g)
        out[f"c{idx}_acc"] = acc.numpy()
        out[f"c{idx}_row"] = row.reshape(-1).numpy()
        out[f"c{idx}_col"] = col.numpy()
        out[f"c{idx}_bias_bf16"] = bits16(bias_bf16)
        out[f"c{idx}_bias_f32"] = bias_f32.numpy()
        out[f"c{idx}_out_none"] = bits16(eager(acc, row, col, None))
        out[f"c{idx}_out_bf16"] = bits16(eager(acc, row, col, bias_bf16))
        out[f"c{idx}_out_f32"] = bits16(eager(acc, row, col, bias_f32))
    np.savez_compressed(OUT / "epilogue_eager.npz", **out)


def golden_gates():
    launcher = REF / "launcher/benchmark_launcher_v14_hires_int8_candidate.py"

    class _Props:
        gcnArchName = "gfx936:sramecc+:xnack-"

    class _Cuda:
        @staticmethod
        def get_device_properties(_d):
            return _Props()

    class _Torch:
        bfloat16, float16, float32, int32, int8 = (torch.bfloat16, torch.float16, torch.float32,
                                                   torch.int32, torch.int8)
        Tensor = torch.Tensor
        dtype = torch.dtype
        cuda = _Cuda()

    ns = {"torch": _Torch, "_vec4_epilogue_enabled": True,
          "_VEC4_EPILOGUE_M": frozenset((11819,)), "_VEC4_EPILOGUE_N": frozenset((5376, 21504, 28672)),
          "_is_gfx936": lambda _t: True, "_exact_quantizer_enabled": True,
          "_EXACT_QUANTIZER_M": frozenset((11819,)), "_EXACT_QUANTIZER_K": frozenset((5376, 7168, 14336))}
    extract(launcher, {"_vec4_epilogue_gate", "_exact_quantizer_gate"}, ns)
    vec4, quant = ns["_vec4_epilogue_gate"], ns["_exact_quantizer_gate"]
    dt = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "i32": torch.int32}

    def T(spec):
        return FakeTensor(tuple(spec["shape"]), dt[spec["dtype"]], contiguous=spec.get("contiguous", True),
                          device=spec.get("device", "cuda:0"), is_cuda=spec.get("is_cuda", True),
                          requires_grad=spec.get("requires_grad", False))

    M, N = 11819, 5376
    acc, row, col = ({"shape": [M, N], "dtype": "i32"}, {"shape": [M], "dtype": "f32"},
                     {"shape": [N], "dtype": "f32"})
    vec4_cases = [
        {"name": "eligible", "acc": acc, "row": row, "col": col},
        {"name": "bias", "acc": acc, "row": row, "col": col, "bias": {"shape": [N], "dtype": "bf16"}},
        {"name": "out_dtype", "acc": acc, "row": row, "col": col, "out_dtype": "f16"},
        {"name": "acc_dtype", "acc": {"shape": [M, N], "dtype": "f16"}, "row": row, "col": col},
        {"name": "row_dtype", "acc": acc, "row": {"shape": [M], "dtype": "bf16"}, "col": col},
        {"name": "col_dtype", "acc": acc, "row": row, "col": {"shape": [N], "dtype": "bf16"}},
        {"name": "not_cuda", "acc": dict(acc, is_cuda=False), "row": row, "col": col},
        {"name": "other_device", "acc": acc, "row": dict(row, device="cuda:1"), "col": col},
        {"name": "acc_strided", "acc": dict(acc, contiguous=False), "row": row, "col": col},
        {"name": "row_strided", "acc": acc, "row": dict(row, contiguous=False), "col": col},
        {"name": "col_strided", "acc": acc, "row": row, "col": dict(col, contiguous=False)},
        {"name": "bad_M", "acc": {"shape": [M - 1, N], "dtype": "i32"}, "row": row, "col": col},
        {"name": "bad_N", "acc": {"shape": [M, N + 1], "dtype": "i32"}, "row": row,
         "col": {"shape": [N + 1], "dtype": "f32"}},
        {"name": "row_shape", "acc": acc, "row": {"shape": [M, 1], "dtype": "f32"}, "col": col},
        {"name": "col_shape", "acc": acc, "row": row, "col": {"shape": [N - 1], "dtype": "f32"}},
        {"name": "acc_3d", "acc": {"shape": [1, M, N], "dtype": "i32"}, "row": row, "col": col},
    ]
    for c in vec4_cases:
        bias = T(c["bias"]) if "bias" in c else None
        c["expect"] = list(vec4(T(c["acc"]), T(c["row"]), T(c["col"]), bias, dt[c.get("out_dtype", "bf16")]))
    x = {"shape": [M, 5376], "dtype": "bf16"}
    quant_cases = [
        {"name": "eligible", "x": x},
        {"name": "stochastic", "x": x, "stochastic_rounding": 1},
        {"name": "dtype", "x": dict(x, dtype="f16")},
        {"name": "device", "x": dict(x, is_cuda=False)},
        {"name": "requires_grad", "x": dict(x, requires_grad=True)},
        {"name": "noncontiguous", "x": dict(x, contiguous=False)},
        {"name": "M", "x": {"shape": [7, 5376], "dtype": "bf16"}},
        {"name": "three_d", "x": {"shape": [1, M, 5376], "dtype": "bf16"}},
        {"name": "K", "x": {"shape": [M, 5377], "dtype": "bf16"}},
    ]
    for c in quant_cases:
        c["expect"] = list(quant(T(c["x"]), c.get("stochastic_rounding", 0)))
    # arch refusal comes last in both gates
    ns["_is_gfx936"] = lambda _t: False
    _Props.gcnArchName = "gfx90a"
    arch = {"vec4": list(vec4(T(acc), T(row), T(col), None, torch.bfloat16)),
            "quant": list(quant(T(x), 0))}
    ns["_vec4_epilogue_enabled"] = False
    ns["_exact_quantizer_enabled"] = False
    disabled = {"vec4": list(vec4(T(acc), T(row), T(col), None, torch.bfloat16)),
                "quant": list(quant(T(x), 0))}
    (OUT / "gate_reasons.json").write_text(json.dumps(
        {"vec4": vec4_cases, "quantizer": quant_cases, "arch": arch, "disabled": disabled}, indent=1))


def golden_attention():
    ns1 = extract(REF / "validation/validate_flash_longseq.py", {"ref_rows"}, {"torch": torch})
    ns2 = extract(REF / "benchmarks/bench_opendas_h3_flash_bshd.py", {"exact_fp32"},
                  {"torch": torch, "DIM": 128})
    out = {}
    for idx, (s, h, seed) in enumerate(((129, 2, 1129), (257, 1, 1257))):
        g = torch.Generator().manual_seed(seed)
        # the reference's production layout: [S, H*128] storage viewed as [1,H,S,128]
        q, k, v = (torch.randn(s, h * 128, generator=g).to(torch.bfloat16).view(1, s, h, 128)
                   .permute(0, 2, 1, 3) for _ in range(3))
        out[f"a{idx}_q"], out[f"a{idx}_k"], out[f"a{idx}_v"] = (bits16(t.contiguous()) for t in (q, k, v))
        out[f"a{idx}_bf16"] = bits16(ns2["exact_fp32"](q, k, v))
        out[f"a{idx}_rows_h0"] = ns1["ref_rows"](q, k, v, 0, 0, s, 128 ** -0.5).numpy()
    np.savez_compressed(OUT / "attention_fp32.npz", **out)


def golden_quantizer_kat():
    """Known answers derived by hand from the reference's comments."""
    kat = [
        # max 127 -> scale exactly 1.0 -> half-integers exercise ties-to-even
        {"name": "round_even_boundaries",
         "x": [127.0, -127.0, 126.5, 125.5, 2.5, 1.5, 0.5, -0.5, -1.5, -2.5, -125.5, -126.5, 0.0],
         "scale_bits": f32bits(1.0),
         "q": [127, -127, 126, 126, 2, 2, 0, 0, -2, -2, -126, -126, 0]},
        # max 63.5 -> scale 0.5 (63.5 * fp32(1/127) rounds to exactly 0.5)
        {"name": "round_even_scale_0.5",
         "x": [63.5, -63.5, 62.5, 1.25, 0.75, 0.25, -0.25, -0.75, -1.25, 0.0],
         "scale_bits": f32bits(0.5),
         "q": [127, -127, 125, 2, 2, 0, 0, -2, -2, 0]},
        {"name": "all_zero", "x": [0.0] * 16, "scale_bits": f32bits(1.0e-30), "q": [0] * 16},
        {"name": "nan_and_infinities", "x": ["nan", "inf", "-inf", 1.0, -1.0, 0.0],
         "scale_bits": 0x7fc00000, "q": [0, 0, 0, 0, 0, 0]},
        # absmax 4.5: multiply-by-reciprocal and true division differ by one ulp
        {"name": "reciprocal_witness_4.5", "x": [4.5, -2.25, 1.0, 0.0],
         "scale_bits": f32bits(float(np.float32(4.5) * np.float32(0.0078740157186985015869140625))),
         "q": None},
        {"name": "infinity_without_nan", "x": ["inf", 3.0, -2.0, 0.0],
         "scale_bits": 0x7f800000, "q": [0, 0, 0, 0]},
    ]
    (OUT / "quantizer_kat.json").write_text(json.dumps(kat, indent=1))


if __name__ == "__main__":
    golden_epilogue()
    golden_gates()
    golden_attention()
    golden_quantizer_kat()
    for p in sorted(OUT.iterdir()):
        print(p.name, p.stat().st_size)
