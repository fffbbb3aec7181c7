"""Gate semantics without a GPU, driven by fake tensors like the reference's own
contract verifier (kernels/int8-epilogue-vec4/verify_v11_contract.py:21-39,81-103).
The expected reasons come from the REFERENCE's gate functions (fixture
tests/golden/gate_reasons.json, generated from the reference launcher)."""
import json
from pathlib import Path

import pytest
import torch

GOLD = Path(__file__).parent / "golden"
DT = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "i32": torch.int32}


class FakeTensor:
    def __init__(self, shape, dtype, *, contiguous=True, device="cuda:0", is_cuda=True,
                 requires_grad=False, stride=None):
        self.shape = tuple(shape)
        self.dtype = dtype
        self.is_cuda = is_cuda
        self.device = torch.device(device) if is_cuda else torch.device("cpu")
        self.requires_grad = requires_grad
        self._contiguous = contiguous
        self._stride = stride
        self.ndim = len(self.shape)

    def is_contiguous(self):
        return self._contiguous

    def dim(self):
        return len(self.shape)

    def numel(self):
        n = 1
        for s in self.shape:
            n *= s
        return n

    def stride(self):
        return self._stride


def T(spec):
    return FakeTensor(spec["shape"], DT[spec["dtype"]], contiguous=spec.get("contiguous", True),
                      device=spec.get("device", "cuda:0"), is_cuda=spec.get("is_cuda", True),
                      requires_grad=spec.get("requires_grad", False))


@pytest.fixture()
def gates(pkg):
    g = pkg.gates.Gates.all_on(load=False)
    g.is_arch = lambda _t: True
    g.audited = lambda _op=None: True
    return g


def test_reasons_match_the_reference_gate_functions(gates):
    gold = json.loads((GOLD / "gate_reasons.json").read_text())
    for c in gold["vec4"]:
        bias = T(c["bias"]) if "bias" in c else None
        got = gates.vec4_epilogue_gate(T(c["acc"]), T(c["row"]), T(c["col"]), bias,
                                       DT[c.get("out_dtype", "bf16")])
        assert list(got) == c["expect"], c["name"]
    for c in gold["quantizer"]:
        got = gates.exact_quantizer_gate(T(c["x"]), c.get("stochastic_rounding", 0))
        assert list(got) == c["expect"], c["name"]
    acc = {"shape": [11819, 5376], "dtype": "i32"}
    row, col = {"shape": [11819], "dtype": "f32"}, {"shape": [5376], "dtype": "f32"}
    x = {"shape": [11819, 5376], "dtype": "bf16"}
    gates.is_arch = lambda _t: False
    assert list(gates.vec4_epilogue_gate(T(acc), T(row), T(col), None, torch.bfloat16)) == gold["arch"]["vec4"]
    assert list(gates.exact_quantizer_gate(T(x))) == gold["arch"]["quant"]
    gates.vec4_epilogue_enabled = False
    gates.exact_quantizer_enabled = False
    assert list(gates.vec4_epilogue_gate(T(acc), T(row), T(col), None, torch.bfloat16)) == gold["disabled"]["vec4"]
    assert list(gates.exact_quantizer_gate(T(x))) == gold["disabled"]["quant"]


def test_audit_refusal_and_b200_whitelists(gates, pkg):
    x = FakeTensor((23638, 3072), torch.bfloat16)
    assert gates.exact_quantizer_gate(x) == (True, "eligible")
    for m in (4096, 23638, 11819, 5909, 5910, 2954, 2955, 109099, 54549, 54550, 27274, 27275,
              13637, 13638):
        assert m in pkg.gates.LOCAL_M
    gates.audited = lambda _op=None: False
    assert gates.exact_quantizer_gate(x) == (False, "audit")
    assert gates.swiglu_quant_gate(FakeTensor((23638, 16384), torch.bfloat16)) == (False, "audit")
    gates.audited = lambda _op=None: True
    assert gates.swiglu_quant_gate(FakeTensor((23638, 16384), torch.bfloat16)) == (True, "eligible")
    assert gates.swiglu_quant_gate(FakeTensor((23638, 16386), torch.bfloat16))[1] == "K"
    v = FakeTensor((3072,), torch.bfloat16)
    assert gates.mod_scale_shift_gate(FakeTensor((23638, 3072), torch.bfloat16), v, v) == (True, "eligible")
    assert gates.mod_scale_shift_gate(FakeTensor((23638, 3072), torch.bfloat16), v,
                                      FakeTensor((3071,), torch.bfloat16))[1] == "vector_shape"
    a8, w8t = FakeTensor((23638, 3072), torch.int8), FakeTensor((3072, 9216), torch.int8)
    assert gates.unpadded_gemm_gate(a8, w8t) == (True, "eligible")
    assert gates.unpadded_gemm_gate(FakeTensor((23637, 3072), torch.int8), w8t)[1] == "MKN"
    rs, cs = FakeTensor((23638,), torch.float32), FakeTensor((9216,), torch.float32)
    w8 = FakeTensor((9216, 3072), torch.int8)
    assert gates.fused_gemm_gate(a8, rs, w8, cs, None, torch.bfloat16) == (True, "eligible")
    assert gates.fused_gemm_gate(a8, rs, w8, cs, FakeTensor((9216,), torch.float16), torch.bfloat16)[1] == "bias_dtype"
    assert gates.fused_gemm_gate(a8, rs, w8, cs, None, torch.float16)[1] == "out_dtype"


def test_startup_invariants(pkg, monkeypatch, tmp_path):
    with pytest.raises(RuntimeError, match="requires H3_INT8_EPILOGUE=1"):
        pkg.gates.Gates(epilogue_vec4=True, epilogue=False, load=False)
    # an enabled feature with an unloadable artifact fails at construction
    monkeypatch.setenv("B2DIT_SO", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="Cannot load required"):
        pkg.gates.Gates(exact_quantizer=True)
    monkeypatch.delenv("B2DIT_SO")
    pkg._lib.load()
    monkeypatch.setenv("H3_INT8_EXACT_QUANTIZER", "1")
    g = pkg.gates.Gates.from_env(load=False)
    assert g.exact_quantizer_enabled and not g.flash_enabled


def test_refusal_counts_and_fallback(gates):
    calls = []
    gates.register_fallbacks(quantize=lambda x, stochastic_rounding=0: calls.append(x.shape) or "fb")
    bad = FakeTensor((7, 3072), torch.bfloat16)
    assert gates.quantize_activation(bad) == "fb"
    assert gates.quantize_activation(FakeTensor((8, 3072), torch.bfloat16)) == "fb"
    assert gates.quantize_activation(bad) == "fb"
    summary = gates.dump_counters()["exact_quantizer"]
    assert summary == {"hits": 0, "fallbacks": 3, "reasons": {"M": 3}}
    # every refused shape is logged once, not only the first per reason
    assert len(gates.counters["exact_quantizer"]._logged) == 2
    g2 = type(gates).all_on(load=False)
    g2.is_arch = lambda _t: True
    g2.audited = lambda _op=None: True
    with pytest.raises(RuntimeError, match="no 'quantize' fallback"):
        g2.quantize_activation(bad)


def test_artifact_audit_table(pkg, tmp_path, monkeypatch):
    import shutil
    so = tmp_path / "libcopy.so"
    shutil.copy(pkg._lib.so_path(), so)
    monkeypatch.setenv("B2DIT_SO", str(so))
    monkeypatch.setattr(pkg._lib, "_lib", None)
    pkg._lib.load()
    assert not pkg._lib.audited()            # no table yet
    pkg._lib.admit(so, note="test")
    assert pkg._lib.audited("quantize_int8_rowwise")
    table = tmp_path / "libcopy.so.audit.json"
    data = json.loads(table.read_text())
    data["artifacts"] = {"0" * 64: {"file": "x"}}
    table.write_text(json.dumps(data))
    assert not pkg._lib.audited()            # unknown hash => refused
    monkeypatch.delenv("B2DIT_SO")
    monkeypatch.setattr(pkg._lib, "_lib", None)
    pkg._lib.load()


def test_flash_gate(pkg, gates):
    A = pkg.attention
    S, H = 23638, 24

    def qkv(shape, stride, **kw):
        return [FakeTensor(shape, torch.bfloat16, stride=stride, **kw) for _ in range(3)]

    sp1 = A.SPContext(0, 1, (S,), S)
    q, k, v = qkv((1, H, S, 128), (S * H * 128, 128, H * 128, 1))
    assert A.flash_gate(gates, q, k, v, H, None, True, {}, sp1) == (True, "eligible", False)
    q, k, v = qkv((1, H, S, 128), (S * H * 384, 128, 3 * H * 128, 1))   # packed qkv projection
    assert A.flash_gate(gates, q, k, v, H, None, True, {}, sp1)[0]
    assert A.flash_gate(gates, q, k, v, H, object(), True, {}, sp1)[1] == "mask"
    assert A.flash_gate(gates, q, k, v, H, None, False, {}, sp1)[1] == "skip_reshape"
    assert A.flash_gate(gates, q, k, v, H, None, True, {"scale": 0.1}, sp1)[1] == "scale"
    assert A.flash_gate(gates, q, k, v, H, None, True, {"enable_gqa": True}, sp1)[1] == "gqa"
    assert A.flash_gate(gates, q, k, v, H, None, True, {}, sp1, torch.float32)[1] == "precision"
    assert A.flash_gate(gates, q, k, v, H, None, True, {}, None)[1] == "sp_world"
    assert A.flash_gate(gates, q, k, v, H, None, True, {}, A.SPContext(0, 3))[1] == "sp_world"
    q2, k2, v2 = qkv((1, H, S, 128), (S * H * 128, S * 128, 128, 1))     # BHSD-contiguous: not admitted
    assert A.flash_gate(gates, q2, k2, v2, H, None, True, {}, sp1)[1] == "layout"
    q3, k3, v3 = qkv((1, H, 131073, 128), (0, 128, H * 128, 1))
    assert A.flash_gate(gates, q3, k3, v3, H, None, True, {}, sp1)[1] == "sequence"
    q4, k4, v4 = qkv((1, H, S, 128), (0, 128, H * 128, 1), requires_grad=True)
    assert A.flash_gate(gates, q4, k4, v4, H, None, True, {}, sp1)[1] == "requires_grad"
    # head-chunk layout: views into the packed all-to-all receive buffer, 8 ranks
    splits = A.expected_splits(109099, 8)
    assert splits[:3] == (13638, 13638, 13638) and splits[3:] == (13637,) * 5
    sp8 = A.SPContext(3, 8, splits, 13637)
    qc, kc, vc = qkv((1, 3, 109099, 128), (0, 384, 3 * 384, 1))
    assert A.flash_gate(gates, qc, kc, vc, 3, None, True, {}, sp8) == (True, "eligible", True)
    bad_sp = A.SPContext(3, 8, splits, 13638)
    assert A.flash_gate(gates, qc, kc, vc, 3, None, True, {}, bad_sp)[1] == "layout"
    gates.head_chunk_overlap_enabled = False
    assert A.flash_gate(gates, qc, kc, vc, 3, None, True, {}, sp8)[1] == "layout"
    gates.is_arch = lambda _t: False
    assert A.flash_gate(gates, q, k, v, H, None, True, {}, sp1)[1] == "arch"
    gates.flash_enabled = False
    assert A.flash_gate(gates, q, k, v, H, None, True, {}, sp1)[1] == "disabled"


def test_head_chunk_choice_fills_the_last_wave():
    """23638 tokens give 93 CTAs per head: one head per launch would leave 55 of 148 SMs idle,
    so fewer, larger chunks are chosen; 109099 tokens (427 CTAs per head) keep the most chunks."""
    import importlib
    import sys
    from pathlib import Path
    sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
    ul = importlib.import_module("dcu-video-dit-turbo_b200").ulysses
    assert [ul.choose_head_chunks(23638, 24 // p) for p in (2, 4, 8)] == [4, 2, 1]
    assert [ul.choose_head_chunks(109099, 24 // p) for p in (2, 4, 8)] == [4, 3, 3]
    assert ul.choose_head_chunks(100, 3) in (1, 3)       # tiny launches: any divisor, never 0
    for heads in (1, 2, 3, 6, 12, 24):
        c = ul.choose_head_chunks(5000, heads)
        assert 1 <= c <= 4 and heads % c == 0
