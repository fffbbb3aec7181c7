"""DiT-block glue kernels (no reference source: this project's conventions) against
the oracle's statement of the same conventions, within bf16 rounding."""
import pytest
import torch

from helpers import bits

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.mark.parametrize("m,c", [(5, 64), (33, 1024), (17, 2048), (129, 3072), (9, 8192)])
def test_layernorm_mod_and_quant(cuda_pkg, ref, m, c):
    g = torch.Generator().manual_seed(m + c)
    x = (torch.randn((m, c), generator=g) * 1.7 + 0.3).to(torch.bfloat16)
    sc = (torch.randn((c,), generator=g) * 0.1).to(torch.bfloat16)
    sh = (torch.randn((c,), generator=g) * 0.1).to(torch.bfloat16)
    want = ref.mod_scale_shift(ref.layer_norm_noaffine(x), sc, sh)
    got = cuda_pkg.ops.layernorm_mod(x.to(DEV), sc.to(DEV), sh.to(DEV)).cpu()
    # fp32 reduction order differs from torch's: allow one bf16 ulp on a few elements
    diff = (got.float() - want.float()).abs()
    assert float(diff.max()) <= 0.04 and float((bits(got) != bits(want)).float().mean()) < 0.02
    # the fused quantizer must equal the oracle quantizer applied to the kernel's own
    # bf16 output, bit for bit
    q, s = cuda_pkg.ops.layernorm_mod_quant(x.to(DEV), sc.to(DEV), sh.to(DEV))
    qr, sr = ref.quantize_int8_rowwise(got)
    assert torch.equal(q.cpu(), qr) and torch.equal(bits(s.cpu()), bits(sr))


@pytest.mark.parametrize("s,h", [(1, 1), (37, 3), (300, 24)])
def test_qk_norm_rope(cuda_pkg, ref, s, h):
    g = torch.Generator().manual_seed(s * 3 + h)
    qkv = torch.randn((s, 3, h, 128), generator=g).to(torch.bfloat16)
    qw = (1 + torch.randn((128,), generator=g) * 0.02).to(torch.bfloat16)
    kw = (1 + torch.randn((128,), generator=g) * 0.02).to(torch.bfloat16)
    pos = torch.stack((torch.arange(s) // 7, torch.arange(s) % 7, torch.arange(s) % 5), -1)
    cos, sin = ref.rope_tables(pos)
    cos2, sin2 = cuda_pkg.block.rope_tables(pos)
    assert torch.equal(cos, cos2) and torch.equal(sin, sin2)
    d = qkv.to(DEV)
    cuda_pkg.ops.qk_norm_rope_(d, qw.to(DEV), kw.to(DEV), cos.to(DEV), sin.to(DEV))
    got = d.cpu()
    want_q = ref.qk_norm_rope(qkv[:, 0], qw, cos, sin)
    want_k = ref.qk_norm_rope(qkv[:, 1], kw, cos, sin)
    assert torch.equal(bits(got[:, 2]), bits(qkv[:, 2]))          # v untouched
    for a, b in ((got[:, 0], want_q), (got[:, 1], want_k)):
        assert float((a.float() - b.float()).abs().max()) <= 0.04
        assert float((bits(a) != bits(b)).float().mean()) < 0.02


@pytest.mark.parametrize("m,c", [(3, 8), (65, 3072), (5, 7)])
def test_gate_residual_bit_exact(cuda_pkg, ref, m, c):
    g = torch.Generator().manual_seed(m * c)
    x = torch.randn((m, c), generator=g).to(torch.bfloat16)
    y = torch.randn((m, c), generator=g).to(torch.bfloat16)
    gate = (torch.randn((c,), generator=g) * 0.1).to(torch.bfloat16)
    xd = x.to(DEV)
    cuda_pkg.ops.gate_residual_(xd, y.to(DEV), gate.to(DEV))
    assert torch.equal(bits(xd.cpu()), bits(ref.gate_residual(x, y, gate)))
