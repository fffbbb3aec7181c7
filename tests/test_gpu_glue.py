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


@pytest.mark.parametrize("s,h,world,chunks", [(37, 24, 1, 1), (37, 24, 2, 1), (50, 24, 4, 2), (19, 24, 8, 3),
                                              (33, 24, 2, 3), (5, 4, 2, 2)])
def test_qk_norm_rope_pack_equals_in_place_then_pack(cuda_pkg, ref, s, h, world, chunks):
    """The fused norm + rotary + all-to-all pack writes exactly the bits of the in-place
    kernel followed by the oracle's pack, and leaves its input untouched."""
    g = torch.Generator().manual_seed(s + h + world + chunks)
    qkv = torch.randn((s, 3, h, 128), generator=g).to(torch.bfloat16)
    qw = (1 + torch.randn((128,), generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    kw = (1 + torch.randn((128,), generator=g) * 0.02).to(torch.bfloat16).to(DEV)
    pos = torch.stack((torch.arange(s) // 7, torch.arange(s) % 7, torch.arange(s) % 5), -1)
    cos, sin = (t.to(DEV) for t in ref.rope_tables(pos))
    src = qkv.to(DEV)
    send = cuda_pkg.ops.qk_norm_rope_pack(src, qw, kw, cos, sin, world, chunks)
    assert tuple(send.shape) == (chunks, world, s, h // (world * chunks), 3, 128)
    assert torch.equal(bits(src.cpu()), bits(qkv))
    in_place = qkv.to(DEV)
    cuda_pkg.ops.qk_norm_rope_(in_place, qw, kw, cos, sin)
    assert torch.equal(bits(send.cpu()), bits(ref.pack_send(in_place.cpu(), world, chunks)))
    with pytest.raises(RuntimeError):
        cuda_pkg.ops.qk_norm_rope_pack(src, qw, kw, cos, sin, 5, 1)


@pytest.mark.parametrize("m,k,world,chunks", [(37, 3072, 2, 1), (50, 3072, 4, 2), (19, 3072, 8, 3), (7, 1024, 1, 1),
                                              (9, 8192, 4, 4), (5, 16384, 2, 1), (3, 64, 2, 2)])
def test_gathered_quantizer_equals_quantizer_of_unpacked_rows(cuda_pkg, ref, m, k, world, chunks):
    """Reading the reverse all-to-all's buffer in place gives the bits of quantising the
    unpacked [M,K] tensor (oracle) - q and scale."""
    g = torch.Generator().manual_seed(m + k + world)
    w = k // (world * chunks)
    recv = (torch.randn((chunks, world, m, w), generator=g) * 3).to(torch.bfloat16)
    recv[0, 0, 0, :] = 0                      # part of a row that is zero
    if m > 2:
        recv[:, :, 2, :] = 0                  # an all-zero row
    q, s = cuda_pkg.ops.quantize_int8_rowwise_gathered(recv.to(DEV))
    rows = ref.unpack_gathered(recv.view(chunks, world, m, 1, w))
    qr, sr = ref.quantize_int8_rowwise(rows)
    assert torch.equal(q.cpu(), qr) and torch.equal(bits(s.cpu()), bits(sr))
    q2, s2 = cuda_pkg.ops.quantize_int8_rowwise(rows.to(DEV))
    assert torch.equal(q2, q) and torch.equal(bits(s2.cpu()), bits(s.cpu()))
    with pytest.raises(RuntimeError):
        cuda_pkg.ops.quantize_int8_rowwise_gathered(recv.to(DEV)[..., :-4])


@pytest.mark.parametrize("m,c", [(3, 8), (65, 3072), (5, 7)])
def test_gate_residual_bit_exact(cuda_pkg, ref, m, c):
    g = torch.Generator().manual_seed(m * c)
    x = torch.randn((m, c), generator=g).to(torch.bfloat16)
    y = torch.randn((m, c), generator=g).to(torch.bfloat16)
    gate = (torch.randn((c,), generator=g) * 0.1).to(torch.bfloat16)
    xd = x.to(DEV)
    cuda_pkg.ops.gate_residual_(xd, y.to(DEV), gate.to(DEV))
    assert torch.equal(bits(xd.cpu()), bits(ref.gate_residual(x, y, gate)))


@pytest.mark.parametrize("shape", [(3, 17, 23, 3), (1, 1, 1, 3), (2, 64, 64, 3), (5, 7, 3)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_images_to_u8_bit_exact(cuda_pkg, ref, shape, dtype):
    """One launch over the clip == the oracle == the per-frame expression evaluated by torch on
    the device; special values follow the documented rule (NaN -> 0)."""
    g = torch.Generator().manual_seed(sum(shape))
    x = (torch.rand(shape, generator=g) * 1.5 - 0.25).to(dtype)
    flat = x.view(-1)
    vals = torch.tensor([0.0, 1.0, 1 / 255, 254.5 / 255, -1e-8, 2.0]).to(dtype)
    k = min(6, flat.numel())
    flat[:k] = vals[:k]
    got = cuda_pkg.ops.images_to_u8(x.to(DEV))
    assert got.dtype == torch.uint8 and got.shape == x.shape
    assert torch.equal(got.cpu(), ref.images_to_u8(x))
    assert torch.equal(got, (x.to(DEV) * 255).clamp(0, 255).byte())
    special = torch.tensor([float("nan"), float("inf"), -float("inf"), 0.5] * 5).to(dtype)
    assert cuda_pkg.ops.images_to_u8(special.to(DEV)).cpu().tolist() == [0, 255, 0, 127] * 5
    # an unaligned view takes the scalar kernel
    y = x.reshape(-1)[1:]
    if y.numel():
        assert torch.equal(cuda_pkg.ops.images_to_u8(y.to(DEV).clone()).cpu(), ref.images_to_u8(y))
    with pytest.raises(RuntimeError):
        cuda_pkg.ops.images_to_u8(x.to(DEV).to(torch.float64))


def test_batched_save_returns_the_per_frame_bytes(cuda_pkg, ref):
    s = cuda_pkg.save.BatchU8Save(enabled=True)
    g = torch.Generator().manual_seed(9)
    clip = torch.rand((4, 36, 64, 3), generator=g)
    host = s.frames_u8(clip.to(DEV), bit_depth=8)
    assert not host.is_cuda and host.is_pinned() and s.hits == 1
    per_frame = torch.stack([(f * 255).clamp(0, 255).byte() for f in clip])
    assert torch.equal(host, per_frame)
    cuda_pkg.ops.check_device_status()
