"""The stand-in extension modules load by file path exactly as the reference's launcher
loads its DSOs (launcher/benchmark_launcher_v14_hires_int8_candidate.py:135-154 in the
reference) and expose the callables it checks for."""
import importlib.util
from pathlib import Path

import pytest
import torch

EXT = Path(__file__).resolve().parents[1] / "dcu-video-dit-turbo_b200" / "ext"
EXPECTED = {
    "h3_exact_rowwise_int8": "quantize_int8_rowwise",
    "h3_hip_epilogue": "epilogue",
    "h3_exact_epilogue_vec4": "epilogue",
    "h3_exact_mod": "mod_scale_shift_",
    "h3_exact_swiglu_quant": "swiglu_quantize_int8_rowwise",
    "h3_flash_attn": "fwd_bhsd",
}


def _load(name):
    spec = importlib.util.spec_from_file_location(name, EXT / f"{name}.py")
    assert spec is not None and spec.loader is not None
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.mark.parametrize("name,attr", sorted(EXPECTED.items()))
def test_loads_by_path_and_has_the_callable(name, attr):
    assert callable(getattr(_load(name), attr))


@pytest.mark.gpu
def test_shim_runs_on_the_gpu():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    x = torch.randn((64, 3072), device="cuda").to(torch.bfloat16)
    q, s = _load("h3_exact_rowwise_int8").quantize_int8_rowwise(x)
    assert q.dtype == torch.int8 and s.shape == (64, 1)
    acc = torch.randint(-1000, 1000, (64, 256), device="cuda", dtype=torch.int32)
    rs, cs = torch.rand(64, device="cuda"), torch.rand(256, device="cuda")
    a = _load("h3_hip_epilogue").epilogue(acc, rs, cs, torch.empty(0, device="cuda", dtype=torch.bfloat16))
    b = _load("h3_exact_epilogue_vec4").epilogue(acc, rs, cs)
    assert torch.equal(a, b)
