"""Batched 8-bit frame conversion: oracle known answers and the eligibility gate (no GPU)."""
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))


def test_oracle_known_answers():
    from oracle import ref_ops as ref
    x = torch.tensor([0.0, 1.0, 0.5, -0.2, 1.7, 0.999, 1 / 255, float("nan"), float("inf"), -float("inf")])
    assert ref.images_to_u8(x).tolist() == [0, 255, 127, 0, 255, 254, 1, 0, 255, 0]   # the cast truncates
    # the product is rounded to the input's own type first: bf16(0.999 * 255) = 255
    assert ref.images_to_u8(torch.tensor([0.999]).to(torch.bfloat16)).tolist() == [255]
    # same expression as the per-frame path it replaces
    g = torch.Generator().manual_seed(5)
    clip = torch.rand((3, 4, 5, 3), generator=g) * 1.4 - 0.2
    per_frame = torch.stack([(f * 255).clamp(0, 255).byte() for f in clip])
    assert torch.equal(ref.images_to_u8(clip), per_frame)


def test_gate_order_and_refusal():
    import importlib
    pkg = importlib.import_module("dcu-video-dit-turbo_b200")
    s = pkg.save.BatchU8Save(enabled=False)
    clip = torch.rand((2, 4, 4, 3))
    assert s.gate(clip, 8) == (False, "disabled")
    s = pkg.save.BatchU8Save(enabled=True)
    assert s.gate(clip, 10) == (False, "bit_depth")
    assert s.gate([clip], 8) == (False, "not_tensor")
    assert s.gate(clip[0], 8) == (False, "rank")
    assert s.gate(torch.rand((2, 4, 4, 4)), 8) == (False, "channels")
    assert s.gate(clip, 8) == (False, "device")                      # CPU tensor
    with pytest.raises(RuntimeError, match="no original writer"):
        s.frames_u8(clip, 8)
    s.register_original_writer(lambda images, depth: "host path")
    assert s.frames_u8(clip, 8) == "host path"
    assert s.fallbacks == {"device": 2} and s.hits == 0
