"""The oracle pinned against the reference: its own eager transcriptions (fixtures
generated from the reference's Python by tests/golden/make_golden.py), hand-derived
known answers from its comments, and an independent scalar C restatement."""
import ctypes
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch

from helpers import bits, epilogue_inputs, quantizer_families, swiglu_families

GOLD = Path(__file__).parent / "golden"


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.astype(np.int16)).view(torch.bfloat16)


def _parse(v):
    return float(v) if isinstance(v, str) else v


def test_quantizer_known_answers(ref):
    for kat in json.loads((GOLD / "quantizer_kat.json").read_text()):
        x = torch.tensor([[_parse(v) for v in kat["x"]]], dtype=torch.float32).to(torch.bfloat16)
        q, s = ref.quantize_int8_rowwise(x)
        got_bits = int(s.view(torch.int32)[0, 0]) & 0xFFFFFFFF
        if kat["name"] == "nan_and_infinities":
            assert math.isnan(float(s[0, 0])), kat["name"]
        else:
            assert got_bits == kat["scale_bits"], (kat["name"], hex(got_bits))
        if kat["q"] is not None:
            assert q[0].tolist() == kat["q"], kat["name"]


def test_reciprocal_witness_differs_from_true_division(ref):
    # kernels/exact-rowwise-int8/quantizer_kernel.hip:68-73: absmax 4.5 is a value where
    # multiply-by-fp32(1/127) and a true fp32 division give different scales
    a = torch.tensor(4.5, dtype=torch.float32)
    assert (a * torch.tensor(ref.INV127, dtype=torch.float32)).view(torch.int32) != \
        (a / 127.0).view(torch.int32)


def test_epilogue_matches_reference_eager(ref):
    z = np.load(GOLD / "epilogue_eager.npz")
    for idx in range(3):
        acc = torch.from_numpy(z[f"c{idx}_acc"])
        row = torch.from_numpy(z[f"c{idx}_row"])
        col = torch.from_numpy(z[f"c{idx}_col"])
        for kind, bias in (("none", None), ("bf16", _bf16(z[f"c{idx}_bias_bf16"])),
                           ("f32", torch.from_numpy(z[f"c{idx}_bias_f32"]))):
            want = _bf16(z[f"c{idx}_out_{kind}"])
            got = ref.epilogue(acc, row, col, bias)
            assert torch.equal(bits(got), bits(want)), (idx, kind)


def test_attention_matches_reference_fp32(ref):
    z = np.load(GOLD / "attention_fp32.npz")
    for idx in range(2):
        q, k, v = (_bf16(z[f"a{idx}_{n}"]) for n in "qkv")
        got = ref.attention_fp32(q, k, v, 128 ** -0.5, row_chunk=64)
        want_rows = torch.from_numpy(z[f"a{idx}_rows_h0"])
        assert (got[0, 0] - want_rows).abs().max() < 2e-6
        want_bf16 = _bf16(z[f"a{idx}_bf16"]).float()
        assert (got - want_bf16).abs().max() < 2e-2  # bf16 rounding of O(1) values
        rows = ref.attention_rows_fp32(q, k, v, 0, 3, 40, 128 ** -0.5)
        assert torch.equal(rows, want_rows[3:40]) or (rows - want_rows[3:40]).abs().max() < 2e-6


def _c_quant(lib, x):
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.int8)
    s = torch.empty((m,), dtype=torch.float32)
    lib.oc_quantize_int8_rowwise(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(q.data_ptr()),
                                 ctypes.c_void_p(s.data_ptr()), ctypes.c_int64(m), ctypes.c_int64(k))
    return q, s


@pytest.mark.parametrize("k", [96, 3072])
def test_c_and_torch_oracles_agree_quantizer(ref, oracle_c, k):
    for name, x in quantizer_families(33, k).items():
        q1, s1 = ref.quantize_int8_rowwise(x)
        q2, s2 = _c_quant(oracle_c, x)
        assert torch.equal(q1, q2), name
        nan1, nan2 = torch.isnan(s1.view(-1)), torch.isnan(s2)
        assert torch.equal(nan1, nan2), name
        assert torch.equal(bits(s1.view(-1))[~nan1], bits(s2)[~nan2]), name


def test_c_and_torch_oracles_agree_epilogue_mod(ref, oracle_c):
    acc, row, col, bias_bf16, bias_f32 = epilogue_inputs(19, 44, 20260810)
    for kind, bias in ((0, None), (1, bias_bf16), (2, bias_f32)):
        out = torch.empty((19, 44), dtype=torch.bfloat16)
        oracle_c.oc_epilogue(ctypes.c_void_p(acc.data_ptr()), ctypes.c_void_p(row.data_ptr()),
                             ctypes.c_void_p(col.data_ptr()),
                             ctypes.c_void_p(bias.data_ptr() if bias is not None else 0), kind,
                             ctypes.c_void_p(out.data_ptr()), ctypes.c_int64(19), ctypes.c_int64(44))
        assert torch.equal(bits(out), bits(ref.epilogue(acc, row, col, bias))), kind
    g = torch.Generator().manual_seed(5)
    x = torch.randn((17, 40), generator=g).to(torch.bfloat16)
    sc = (torch.randn((40,), generator=g) * 0.1).to(torch.bfloat16)
    sh = (torch.randn((40,), generator=g) * 0.1).to(torch.bfloat16)
    want = ref.mod_scale_shift(x, sc, sh)
    y = x.clone()
    oracle_c.oc_mod_scale_shift(ctypes.c_void_p(y.data_ptr()), ctypes.c_void_p(sc.data_ptr()),
                                ctypes.c_void_p(sh.data_ptr()), ctypes.c_int64(17), ctypes.c_int64(40))
    assert torch.equal(bits(y), bits(want))


def test_c_and_torch_oracles_agree_swiglu(ref, oracle_c):
    # expf differs between libm and torch's vectorised exp by at most an ulp, which can
    # flip a bf16 rounding: require equality on the deterministic families and allow a
    # vanishing mismatch rate (<= 1e-4, one int8 step) on the random one.
    for name, x in swiglu_families(21, 64).items():
        q1, s1 = ref.swiglu_quantize_int8_rowwise(x)
        m, k = q1.shape
        q2 = torch.empty((m, k), dtype=torch.int8)
        s2 = torch.empty((m,), dtype=torch.float32)
        oracle_c.oc_swiglu_quantize(ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(q2.data_ptr()),
                                    ctypes.c_void_p(s2.data_ptr()), ctypes.c_int64(m),
                                    ctypes.c_int64(k), ctypes.c_void_p(0))
        diff = (q1.int() - q2.int()).abs()
        assert int(diff.max()) <= 1, name
        assert float((diff != 0).float().mean()) <= 1e-4, name


def test_reciprocal_multiply_is_exact_for_every_reachable_scale(oracle_c):
    """The CUDA quantizer multiplies by rn(1/scale) instead of dividing.  Exhaustive
    over every bf16 x and every bf16 scale from bf16(1e-30) (the scale floor) to +inf."""
    lo = int(torch.tensor(1e-30).to(torch.bfloat16).view(torch.int16)) & 0xFFFF
    fx, fs = ctypes.c_uint32(), ctypes.c_uint32()
    bad = oracle_c.oc_recip_mismatches(ctypes.c_uint32(lo), ctypes.c_uint32(0x7F80),
                                       ctypes.byref(fx), ctypes.byref(fs))
    assert bad == 0, (hex(fx.value), hex(fs.value))


def test_int8_mm_and_linear_compose(ref):
    g = torch.Generator().manual_seed(3)
    x = torch.randn((24, 64), generator=g).to(torch.bfloat16)
    w = torch.randint(-127, 128, (16, 64), dtype=torch.int8, generator=g)
    ws = torch.rand((16,), generator=g) * 0.01 + 1e-4
    b = torch.randn((16,), generator=g).to(torch.bfloat16)
    q, s = ref.quantize_int8_rowwise(x)
    acc = ref.int8_mm(q, w)
    assert torch.equal(acc, (q.long() @ w.long().T).int())
    out = ref.int8_linear(x, w, ws, b)
    assert torch.equal(bits(out), bits(ref.epilogue(acc, s.view(-1), ws, b)))
    with pytest.raises(ValueError):
        ref.int8_linear(x[:, :32], w, ws, b)


def test_empty_inputs(ref):
    q, s = ref.quantize_int8_rowwise(torch.empty((3, 0), dtype=torch.bfloat16))
    assert q.shape == (3, 0) and torch.all(s == 1e-30)
    q, s = ref.quantize_int8_rowwise(torch.empty((0, 8), dtype=torch.bfloat16))
    assert q.shape == (0, 8) and s.shape == (0, 1)


def test_ulysses_single_process_model(ref):
    g = torch.Generator().manual_seed(1)
    for world, seq in ((2, 23), (4, 30), (8, 43)):
        splits = ref.ulysses_splits(seq, world)
        assert sum(splits) == seq and max(splits) - min(splits) <= 1
        shards = [torch.randn((n, 8, 4), generator=g) for n in splits]
        heads = ref.sequence_to_heads_all(shards)
        assert all(h.shape == (seq, 8 // world, 4) for h in heads)
        back = ref.heads_to_sequence_all(heads, splits)
        assert all(torch.equal(a, b) for a, b in zip(shards, back))
