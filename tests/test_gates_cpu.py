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


def test_attention_wired_as_the_host_calls_it(pkg, gates, monkeypatch):
    """The launcher swap `optimized_attention = lambda *a, **k: attention(*a, gates=g, **k)`:
    the host passes `transformer_options`, never `sp_context`.  A single-GPU host (no
    sequence-parallel state in the options) and a sequence-parallel host must both reach the
    kernel; a host without options, or one whose resolved precision is fp32 although the
    argument is None, must reach the registered original attention."""
    A = pkg.attention
    S, H = 23638, 24
    launched, fell_back = [], []
    monkeypatch.setattr(A.ops, "fwd_bhsd", lambda q, k, v, scale: launched.append(scale) or "flash")
    monkeypatch.setattr(A.ops, "check_device_status", lambda device=None: None)
    monkeypatch.setattr(A.torch.cuda, "synchronize", lambda device=None: None)
    gates.register_fallbacks(attention=lambda q, k, v, heads, **kw: fell_back.append(sorted(kw)) or "host")
    host_attention = lambda *a, **k: A.attention(*a, gates=gates, **k)      # INTEGRATION.md wiring
    q, k, v = (FakeTensor((1, H, S, 128), torch.bfloat16, stride=(S * H * 128, 128, H * 128, 1))
               for _ in range(3))
    out = host_attention(q, k, v, H, skip_reshape=True, skip_output_reshape=True, transformer_options={})
    assert out == "flash" and len(launched) == 1 and gates.counters["flash"].hits == 1
    # sequence-parallel state travels inside transformer_options
    splits = A.expected_splits(109099, 8)
    qc, kc, vc = (FakeTensor((1, 3, 109099, 128), torch.bfloat16, stride=(0, 384, 3 * 384, 1)) for _ in range(3))
    opts = {A.SP_OPTIONS_KEY: {"rank": 3, "world_size": 8, "sequence_splits": splits, "local_length": 13637}}
    assert host_attention(qc, kc, vc, 3, skip_reshape=True, skip_output_reshape=True,
                          transformer_options=opts) == "flash"
    assert gates.flash_head_chunk_calls == 1
    opts_obj = {A.SP_OPTIONS_KEY: A.SPContext(3, 8, splits, 13637)}
    assert host_attention(qc, kc, vc, 3, skip_reshape=True, skip_output_reshape=True,
                          transformer_options=opts_obj) == "flash"
    # no options at all: refused like the reference (sp_world), original arguments forwarded
    assert host_attention(q, k, v, H, skip_reshape=True) == "host"
    assert gates.counters["flash"].fallbacks["sp_world"] == 1
    assert "attn_precision" in fell_back[-1] and "skip_output_reshape" in fell_back[-1]
    # host-resolved precision: a forced fp32 upcast with attn_precision=None is refused
    gates.precision_resolver = lambda attn_precision, dtype: torch.float32
    assert host_attention(q, k, v, H, skip_reshape=True, transformer_options={}) == "host"
    assert gates.counters["flash"].fallbacks["precision"] == 1
    gates.precision_resolver = None
    # a host with its own place for the state registers a resolver
    gates.context_resolver = lambda options: A.SPContext(0, 2, A.expected_splits(S, 2), 11819)
    assert host_attention(q, k, v, H, skip_reshape=True, skip_output_reshape=True) == "flash"
    assert len(launched) == 4


def test_every_input_the_wrappers_reject_is_a_counted_refusal(gates):
    """Reasons in front of MKN / arch for the two GEMM gates: layouts and devices that
    ops.int_mm / ops.int8_gemm_dequant would raise on go to the fallback instead."""
    a8 = FakeTensor((23638, 3072), torch.int8, stride=(3072, 1))
    w8t = FakeTensor((3072, 9216), torch.int8, stride=(1, 3072))
    assert gates.unpadded_gemm_gate(a8, w8t) == (True, "eligible")
    assert gates.unpadded_gemm_gate(a8, FakeTensor((3072, 9216), torch.int8, stride=(9216, 1)))[1] == "weight_layout"
    assert gates.unpadded_gemm_gate(FakeTensor((23638, 3072), torch.int8, contiguous=False), w8t)[1] == "noncontiguous"
    assert gates.unpadded_gemm_gate(a8, FakeTensor((3072, 9216), torch.int8, device="cuda:1"))[1] == "device_mismatch"
    rs, cs = FakeTensor((23638,), torch.float32), FakeTensor((9216,), torch.float32)
    w8 = FakeTensor((9216, 3072), torch.int8)
    ok_bias = FakeTensor((9216,), torch.bfloat16)
    assert gates.fused_gemm_gate(a8, rs, w8, cs, ok_bias, torch.bfloat16) == (True, "eligible")
    assert gates.fused_gemm_gate(a8, rs, FakeTensor((9216, 3072), torch.int8, device="cuda:1"), cs, None,
                                 torch.bfloat16)[1] == "device_mismatch"
    assert gates.fused_gemm_gate(a8, rs, w8, cs, FakeTensor((9216,), torch.bfloat16, device="cuda:1"),
                                 torch.bfloat16)[1] == "bias_device"
    assert gates.fused_gemm_gate(a8, rs, w8, cs, FakeTensor((9216,), torch.bfloat16, is_cuda=False),
                                 torch.bfloat16)[1] == "bias_device"
    assert gates.fused_gemm_gate(a8, rs, w8, cs, FakeTensor((9216,), torch.bfloat16, contiguous=False),
                                 torch.bfloat16)[1] == "bias_noncontiguous"
    assert gates.fused_gemm_gate(a8, rs, w8, cs, FakeTensor((9215,), torch.bfloat16), torch.bfloat16)[1] == "bias_shape"
    # the refusal is counted and served by the host's GEMM
    gates.register_fallbacks(int_mm=lambda a, wt: "host_gemm")
    assert gates.int8_matmul(a8, FakeTensor((3072, 9216), torch.int8, stride=(9216, 1))) == "host_gemm"
    assert gates.dump_counters()["unpadded_gemm"]["reasons"] == {"weight_layout": 1}


def test_convrot_is_a_counted_refusal_served_by_the_host_rotation(pkg, gates):
    """convrot=True: group-size check as in the reference, then the rotation goes to the
    host's helper (counted under `convrot`) and the rotated activation enters the gated path."""
    lin = pkg.linear
    x = torch.ones((4, 512), dtype=torch.bfloat16)
    w = torch.ones((8, 512), dtype=torch.int8)
    ws = torch.ones((8,))
    with pytest.raises(ValueError, match="ConvRot group size 384 does not divide input features 512"):
        lin.int8_linear(x, w, ws, convrot=True, convrot_groupsize=384, gates=gates)
    with pytest.raises(RuntimeError, match="no 'convrot_rotate' fallback"):
        lin.int8_linear(x, w, ws, convrot=True, gates=gates)
    seen = []

    class Stop(Exception):
        pass

    def quantize(x2d, stochastic_rounding=0):
        seen.append(("quantize", tuple(x2d.shape), float(x2d[0, 0])))
        raise Stop

    gates.register_fallbacks(convrot_rotate=lambda t, group: seen.append(("rotate", group)) or t * 2,
                             quantize=quantize)
    with pytest.raises(Stop):
        lin.int8_linear(x, w, ws, convrot=True, convrot_groupsize=256, gates=gates)
    assert seen == [("rotate", 256), ("quantize", (4, 512), 2.0)]
    assert gates.dump_counters()["convrot"]["reasons"] == {"convrot": 2}


def test_audit_table_is_parsed_once_until_it_changes(pkg, tmp_path, monkeypatch):
    import shutil
    so = tmp_path / "libcopy2.so"
    shutil.copy(pkg._lib.so_path(), so)
    monkeypatch.setenv("B2DIT_SO", str(so))
    monkeypatch.setattr(pkg._lib, "_lib", None)
    pkg._lib.load()
    pkg._lib.admit(so, note="test")
    reads = []
    real = json.loads
    monkeypatch.setattr(pkg._lib.json, "loads", lambda text: reads.append(1) or real(text))
    assert all(pkg._lib.audited("flash_fwd") for _ in range(50))
    assert len(reads) == 1
    pkg._lib.refresh_audit()
    assert pkg._lib.audited() and len(reads) == 2
    monkeypatch.undo()
    monkeypatch.setattr(pkg._lib, "_lib", None)
    pkg._lib.refresh_audit()
    pkg._lib.load()


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
