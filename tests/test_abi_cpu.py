"""The C-ABI library without a GPU: it loads, exports every symbol the header
declares, and rejects bad arguments with a status code before any launch."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _declared_symbols():
    text = (ROOT / "include" / "b2dit.h").read_text()
    return sorted(set(re.findall(r"\b(b2_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg._lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 17
    for name in declared:
        assert hasattr(lib, name), name
        assert name in pkg._lib.SYMBOLS, f"{name} has no ctypes prototype"
    assert lib.b2_version() == pkg._lib.ABI_VERSION


def test_status_strings(pkg):
    lib = pkg._lib.load()
    names = [lib.b2_status_string(i).decode() for i in range(9)]
    assert names == ["OK", "BAD_DTYPE", "BAD_SHAPE", "BAD_STRIDE", "NOT_WHITELISTED",
                     "LAUNCH_FAILED", "TIMEOUT", "NULL_POINTER", "TOO_LARGE"]


def test_argument_validation_precedes_launch(pkg):
    """Every call below must be refused on the host: no CUDA device exists here."""
    lib = pkg._lib.load()
    P = ctypes.c_void_p
    fake = P(0x1000)   # 16-byte aligned, never dereferenced
    odd = P(0x1001)
    assert lib.b2_quantize_int8_rowwise(fake, fake, fake, -1, 8, None) == 2
    assert lib.b2_quantize_int8_rowwise(None, fake, fake, 4, 8, None) == 7
    assert lib.b2_quantize_int8_rowwise(odd, fake, fake, 4, 8, None) == 3
    assert lib.b2_quantize_int8_rowwise(fake, fake, fake, 0, 8, None) == 0   # empty is legal
    assert lib.b2_swiglu_quantize_int8_rowwise(fake, fake, fake, 0, 0, None) == 0
    assert lib.b2_epilogue(fake, fake, fake, None, 3, fake, 4, 4, None) == 1
    assert b"bias must be none, bfloat16, or float32" in lib.b2_last_error()
    assert lib.b2_epilogue(fake, fake, fake, None, 1, fake, 4, 4, None) == 7
    assert lib.b2_epilogue(fake, fake, fake, None, 0, fake, 0, 4, None) == 0
    assert lib.b2_epilogue_vec4(fake, None, fake, fake, 4, 4, None) == 7
    assert lib.b2_mod_scale_shift(None, fake, fake, 4, 4, None) == 7
    assert lib.b2_int8_gemm(fake, fake, fake, 128, 128, 100, None) == 4      # K % 16
    assert lib.b2_int8_gemm(fake, fake, fake, 128, 130, 128, None) == 4      # N % 4
    assert lib.b2_int8_gemm(odd, fake, fake, 128, 128, 128, None) == 3
    assert lib.b2_int8_gemm(fake, fake, fake, 128, 128, 0, None) == 2
    assert lib.b2_int8_gemm_dequant(fake, fake, fake, fake, None, 7, fake, 8, 8, 16, None) == 1
    assert lib.b2_int8_gemm_dequant(fake, fake, fake, fake, None, 0, fake, 8, 12, 16, None) == 4
    assert lib.b2_int8_linear(fake, 9, fake, fake, None, 0, fake, fake, fake, 8, 8, 16, None) == 1
    s = [0, 128, 128 * 4]
    assert lib.b2_flash_fwd(fake, fake, fake, fake, 1, 4, 0, *s, *s, *s, 0.1, None) == 2
    assert lib.b2_flash_fwd(fake, fake, fake, fake, 1, 4, 16, *s, *s, *s, float("nan"), None) == 2
    assert b"softmax_scale must be finite and positive" in lib.b2_last_error()
    assert lib.b2_flash_fwd(fake, fake, fake, fake, 1, 4, 16, *s, *s, *s, -1.0, None) == 2
    bad = [0, 100, 512]
    assert lib.b2_flash_fwd(fake, fake, fake, fake, 1, 4, 16, *bad, *s, *s, 0.1, None) == 3
    assert lib.b2_flash_fwd(odd, fake, fake, fake, 1, 4, 16, *s, *s, *s, 0.1, None) == 3
    assert lib.b2_layernorm_mod(fake, fake, fake, fake, 4, 12, 1e-6, None) == 4
    assert lib.b2_qk_norm_rope(fake, fake, fake, fake, fake, 4, 0, 1e-6, None) == 2
    assert lib.b2_gate_residual(fake, None, fake, 4, 8, None) == 7
    # peer exchange: tables are checked entry by entry before anything is launched
    two = (P * 2)(0x1000, 0x2000)
    assert lib.b2_qk_norm_rope_scatter(fake, two, fake, fake, fake, fake, 4, 24, 2, 1, 0, 8, 1e-6, None) == 3   # aliases the input
    assert lib.b2_qk_norm_rope_scatter(P(0x3000), two, fake, fake, fake, fake, 4, 24, 5, 1, 0, 8, 1e-6, None) == 2
    assert lib.b2_qk_norm_rope_scatter(P(0x3000), two, fake, fake, fake, fake, 4, 24, 2, 1, 6, 8, 1e-6, None) == 2
    assert b"do not fit a sequence" in lib.b2_last_error()
    assert lib.b2_qk_norm_rope_scatter(P(0x3000), (P * 2)(0x1000, 0), fake, fake, fake, fake, 4, 24, 2, 1, 0, 8,
                                       1e-6, None) == 7
    assert lib.b2_qk_norm_rope_scatter(P(0x3000), (P * 2)(0x1000, 0x2004), fake, fake, fake, fake, 4, 24, 2, 1, 0,
                                       8, 1e-6, None) == 3
    assert lib.b2_qk_norm_rope_scatter(P(0x3000), (P * 2)(0x1000, 0x3000), fake, fake, fake, fake, 4, 24, 2, 1, 0,
                                       8, 1e-6, None) == 3
    assert lib.b2_qk_norm_rope_scatter(P(0x3000), two, fake, fake, fake, fake, 0, 24, 2, 1, 0, 8, 1e-6, None) == 0
    assert lib.b2_copy_segments(two, two, (ctypes.c_int64 * 2)(16, 24), 2, None) == 2
    assert lib.b2_copy_segments(two, two, (ctypes.c_int64 * 2)(0, 0), 2, None) == 0     # nothing to copy, nothing launched
    assert lib.b2_copy_segments(None, two, (ctypes.c_int64 * 2)(16, 16), 2, None) == 7
    assert lib.b2_copy_segments(two, two, (ctypes.c_int64 * 2)(16, 16), 9, None) == 2
    assert lib.b2_peer_alloc(-1, ctypes.byref(P())) == 2
    assert lib.b2_peer_alloc(16, None) == 7
    assert lib.b2_peer_export(None, fake, 64) == 7
    assert lib.b2_peer_open(fake, 12, ctypes.byref(P())) == 2
    assert lib.b2_peer_free(None) == 0 and lib.b2_peer_close(None) == 0


def test_missing_library_fails_loudly(pkg, tmp_path):
    with pytest.raises(RuntimeError, match="Cannot load required"):
        pkg._lib.load(tmp_path / "missing_libb2dit.so")
    # a shared object without the expected symbols is refused too
    import subprocess
    src = tmp_path / "stub.c"
    src.write_text("int b2_version(void) { return 1; }\n")
    so = tmp_path / "libstub.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-o", str(so), str(src)], check=True)
    with pytest.raises(RuntimeError, match="lacks"):
        pkg._lib.load(so)
    pkg._lib.load()  # restore the real one


def test_ops_reject_cpu_tensors(pkg):
    import torch
    x = torch.zeros((4, 8), dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="CUDA"):
        pkg.ops.quantize_int8_rowwise(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        pkg.ops.mod_scale_shift_(x, x[0], x[0])
    with pytest.raises(RuntimeError):
        pkg.ops.fwd_bhsd(x, x, x, 0.1)
