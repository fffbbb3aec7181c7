"""ctypes loader for libb2dit.so with the artifact audit.

The launcher spec this mirrors loads each operator DSO by explicit path at
start-up and raises if it is missing or lacks the expected symbol
(launcher/benchmark_launcher_v14_hires_int8_candidate.py:135-154, :840-860 in the
reference); the artifact-hash audit is the reference paper's
SUBSTITUTE(op, shape, artifact) rule (paper/draft.md:88-97): an artifact whose
sha256 is not in the audit table is never substituted.
"""
from __future__ import annotations

import ctypes
import hashlib
import json
import os
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEFAULT_SO = HERE / "libb2dit.so"

# name -> (restype, argtypes); must list every symbol include/b2dit.h declares
_vp, _i64, _i32, _f32, _int = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float, ctypes.c_int
SYMBOLS = {
    "b2_version": (_int, []),
    "b2_last_error": (ctypes.c_char_p, []),
    "b2_status_string": (ctypes.c_char_p, [_int]),
    "b2_check_device_status": (_int, [_vp]),
    "b2_selftest_bounded_wait": (_int, [_vp]),
    "b2_quantize_int8_rowwise": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "b2_epilogue": (_int, [_vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _vp]),
    "b2_epilogue_vec4": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _vp]),
    "b2_mod_scale_shift": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "b2_swiglu_quantize_int8_rowwise": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
    "b2_int8_gemm": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b2_int8_gemm_dequant": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]),
    "b2_int8_gemm_dequant_residual": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b2_int8_gemm_dequant_swiglu": (_int, [_vp, _vp, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]),
    "b2_int8_linear": (_int, [_vp, _int, _vp, _vp, _vp, _int, _vp, _vp, _vp, _i64, _i64, _i64, _vp]),
    "b2_int8_linear_noalloc": (_int, [_vp, _int, _vp, _vp, _vp, _int, _vp, _i64, _i64, _i64, _vp]),
    "b2_flash_fwd": (_int, [_vp, _vp, _vp, _vp, _i32, _i32, _i32] + [_i64] * 9 + [_f32, _vp]),
    "b2_layernorm_mod": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _vp]),
    "b2_layernorm_mod_quant": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32, _vp]),
    "b2_qk_norm_rope": (_int, [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _vp]),
    "b2_qk_norm_rope_pack": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _f32, _vp]),
    "b2_quantize_int8_rowwise_gathered": (_int, [_vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b2_peer_alloc": (_int, [_i64, _vp]),
    "b2_peer_free": (_int, [_vp]),
    "b2_peer_export": (_int, [_vp, _vp, _i32]),
    "b2_peer_open": (_int, [_vp, _i32, _vp]),
    "b2_peer_close": (_int, [_vp]),
    "b2_qk_norm_rope_scatter": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _i64, _i64, _f32, _vp]),
    "b2_copy_segments": (_int, [_vp, _vp, _vp, _i32, _vp]),
    "b2_images_to_u8": (_int, [_vp, _i32, _vp, _i64, _vp]),
    "b2_gate_residual": (_int, [_vp, _vp, _vp, _i64, _i64, _vp]),
}

ABI_VERSION = 1

_lib = None
_lib_path: Path | None = None
_lib_sha256: str | None = None


def so_path() -> Path:
    return Path(os.environ.get("B2DIT_SO", str(DEFAULT_SO)))


def audit_path() -> Path:
    return Path(os.environ.get("B2DIT_AUDIT", str(so_path()) + ".audit.json"))


def sha256_file(path: Path) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 20), b""):
            h.update(chunk)
    return h.hexdigest()


def load(path: str | os.PathLike | None = None):
    """Load the library (once).  Raises RuntimeError when it is missing, has the
    wrong ABI version or lacks a declared symbol: never a silent fallback."""
    global _lib, _lib_path, _lib_sha256
    p = Path(path) if path is not None else so_path()
    if _lib is not None and _lib_path == p:
        return _lib
    if not p.exists():
        raise RuntimeError(
            f"Cannot load required B200 DiT kernel library from {p}: build it with "
            f"`python {HERE / 'build.py'}` (there is no eager or CPU fallback)")
    try:
        lib = ctypes.CDLL(str(p))
    except OSError as exc:
        raise RuntimeError(f"Cannot load required B200 DiT kernel library from {p}: {exc}") from exc
    for name, (restype, argtypes) in SYMBOLS.items():
        fn = getattr(lib, name, None)
        if fn is None:
            raise RuntimeError(f"B200 DiT kernel library lacks {name}: {p}")
        fn.restype = restype
        fn.argtypes = argtypes
    if lib.b2_version() != ABI_VERSION:
        raise RuntimeError(f"B200 DiT kernel library ABI {lib.b2_version()} != {ABI_VERSION}: {p}")
    _lib, _lib_path, _lib_sha256 = lib, p, sha256_file(p)
    return lib


def loaded_sha256() -> str:
    load()
    return _lib_sha256  # type: ignore[return-value]


def admit(path: str | os.PathLike | None = None, note: str = "") -> dict:
    """Record the artifact's sha256 in its audit table (done by the build step once
    the artifact has been produced from the audited sources)."""
    p = Path(path) if path is not None else so_path()
    table_path = Path(str(p) + ".audit.json") if path is not None else audit_path()
    table = {"artifacts": {}}
    if table_path.exists():
        try:
            table = json.loads(table_path.read_text())
        except json.JSONDecodeError:
            table = {"artifacts": {}}
    digest = sha256_file(p)
    table.setdefault("artifacts", {})[digest] = {"file": p.name, "abi": ABI_VERSION, "note": note}
    table_path.write_text(json.dumps(table, indent=1, sort_keys=True))
    refresh_audit()
    return table


# (audit table path, its mtime in ns, its size, artifact digest) -> the artifact's table entry
_audit_cache: tuple | None = None


def refresh_audit() -> None:
    """Forget the cached audit entry (the next `audited()` reads the table again)."""
    global _audit_cache
    _audit_cache = None


def _audit_entry():
    """The loaded artifact's entry in the audit table, or None.  Gated calls ask this several
    times per operator call, so the table is parsed once and kept until the file changes
    (one `stat` per question instead of a read and a JSON parse)."""
    global _audit_cache
    digest = loaded_sha256()
    path = audit_path()
    st = os.stat(path)
    key = (str(path), st.st_mtime_ns, st.st_size, digest)
    if _audit_cache is None or _audit_cache[0] != key:
        table = json.loads(path.read_text())
        _audit_cache = (key, table.get("artifacts", {}).get(digest))
    return _audit_cache[1]


def audited(op: str | None = None) -> bool:
    """True iff the loaded artifact's sha256 is in the audit table."""
    try:
        entry = _audit_entry()
    except (RuntimeError, OSError, json.JSONDecodeError):
        return False
    if entry is None:
        return False
    ops = entry.get("ops")
    return ops is None or op is None or op in ops


def check(status: int, what: str = "") -> None:
    """Turn a non-zero status into the RuntimeError the reference's TORCH_CHECKs raise."""
    if status == 0:
        return
    lib = load()
    msg = lib.b2_last_error().decode(errors="replace")
    name = lib.b2_status_string(status).decode()
    raise RuntimeError(f"{what or 'b2dit'}: {name}: {msg}")
