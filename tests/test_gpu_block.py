"""One DiT block on the GPU against the CPU oracle's block (small token counts), and
properties at the benchmark's full token count."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cpu_params(p):
    return {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in p.items()}


@pytest.mark.parametrize("tokens", [300, 1000])
def test_block_matches_oracle_block(cuda_pkg, ref, tokens):
    pkg = cuda_pkg
    params = pkg.block.make_block_params(seed=3, device=DEV)
    cos, sin = pkg.block.rope_tables(pkg.block.grid_positions(tokens))
    g = torch.Generator().manual_seed(tokens)
    x = torch.randn((tokens, 3072), generator=g).to(torch.bfloat16)
    blk = pkg.block.DiTBlock(params)
    got = blk.forward(x.to(DEV), cos.to(DEV), sin.to(DEV)).cpu()
    pkg.ops.check_device_status()
    want = ref.dit_block(x, _cpu_params(params), cos, sin)
    assert torch.isfinite(got.float()).all()
    # The oracle block uses fp32 attention and torch's reduction order in the norms, the
    # kernels bf16-P flash attention and their own order: a quality gate, not a bit gate.
    # The reference publishes no block-level threshold (its 32.8 dB / 26.9 dB figures are
    # whole-video numbers); 50 dB is this project's conservative choice.
    assert ref.psnr(want, got) >= 50.0, ref.psnr(want, got)
    # input is not modified, and the call is deterministic
    got2 = blk.forward(x.to(DEV), cos.to(DEV), sin.to(DEV)).cpu()
    assert torch.equal(got, got2)


def test_block_full_token_count_properties(cuda_pkg):
    """Benchmark config 4 size (23638 tokens): finite, deterministic, and invariant to
    splitting the token dimension of every row-local stage (rows are independent), which
    is what makes the multi-GPU token sharding exact."""
    pkg = cuda_pkg
    T = 23638
    params = pkg.block.make_block_params(seed=5, device=DEV)
    cos, sin = pkg.block.rope_tables(pkg.block.grid_positions(T))
    cos, sin = cos.to(DEV), sin.to(DEV)
    x = torch.randn((T, 3072), device=DEV).to(torch.bfloat16)
    blk = pkg.block.DiTBlock(params)
    y = blk.forward(x, cos, sin)
    assert torch.isfinite(y.float()).all()
    assert torch.equal(y, blk.forward(x, cos, sin))
    ops, p = pkg.ops, params
    q8, s = ops.layernorm_mod_quant(x, p["scale1"], p["shift1"])
    full = ops.int8_gemm_dequant(q8, s.view(-1), p["wq_qkv"], p["ws_qkv"], p["b_qkv"])
    cut = 11819
    parts = []
    for sl in (slice(0, cut), slice(cut, T)):
        q8p, sp_ = ops.layernorm_mod_quant(x[sl].contiguous(), p["scale1"], p["shift1"])
        parts.append(ops.int8_gemm_dequant(q8p, sp_.view(-1), p["wq_qkv"], p["ws_qkv"], p["b_qkv"]))
    assert torch.equal(full, torch.cat(parts))
    pkg.ops.check_device_status()


def test_graphed_block_equals_eager_block(cuda_pkg):
    pkg = cuda_pkg
    T = 1500
    params = pkg.block.make_block_params(seed=9, device=DEV)
    cos, sin = pkg.block.rope_tables(pkg.block.grid_positions(T))
    cos, sin = cos.to(DEV), sin.to(DEV)
    blk = pkg.block.DiTBlock(params)
    x1 = torch.randn((T, 3072), device=DEV).to(torch.bfloat16)
    x2 = torch.randn((T, 3072), device=DEV).to(torch.bfloat16)
    graphed = pkg.block.GraphedBlock(blk, x1, cos, sin)
    assert graphed.launches_per_replay == 10
    for x in (x1, x2, x1):
        want = blk.forward(x, cos, sin)
        got = graphed(x).clone()
        assert torch.equal(got, want)
    pkg.ops.check_device_status()
