"""b2_int8_linear_noalloc: the INT8 linear for callers that cannot hand the library any
scratch memory (a host whose pool owns the whole device, a plugin that only gets input and
output buffers).  Its scratch is a fixed array inside the library, so this test checks what
such a caller relies on: called straight through the C ABI with nothing but inputs and an
output buffer, it returns exactly the bits of b2_int8_linear with caller scratch - on the
first call, and again on a second call that finds the previous call's data in the array.

Named test_zz_* so that it is collected after every other test file."""
import ctypes

import pytest
import torch

DEV = "cuda:0"
P = ctypes.c_void_p


def test_sizes_beyond_the_builtin_scratch_are_refused_on_the_host(pkg):
    """No GPU needed: the size check comes before any CUDA call."""
    lib = pkg._lib.load()
    fake = P(0x1000)
    too_many_rows = lib.b2_int8_linear_noalloc(fake, 0, fake, fake, None, 0, fake, 65537, 64, 64, None)
    assert too_many_rows == 8 and b"exceeds the built-in scratch" in lib.b2_last_error()
    too_many_bytes = lib.b2_int8_linear_noalloc(fake, 0, fake, fake, None, 0, fake, 8192, 64, 8192, None)
    assert too_many_bytes == 8
    assert lib.b2_int8_linear_noalloc(fake, 5, fake, fake, None, 0, fake, 8, 8, 16, None) == 1
    assert lib.b2_int8_linear_noalloc(fake, 0, fake, fake, None, 0, fake, 8, 12, 16, None) == 4
    assert lib.b2_int8_linear_noalloc(fake, 0, fake, fake, None, 0, fake, 0, 8, 16, None) == 0


@pytest.mark.gpu
def test_noalloc_linear_equals_scratch_linear_on_two_calls_in_a_row(cuda_pkg, ref):
    pkg = cuda_pkg
    lib = pkg._lib.load()
    stream = torch.cuda.current_stream(DEV).cuda_stream
    g = torch.Generator().manual_seed(77)
    # two different problems so the second call meets stale data from the first in the
    # shared array: a plain linear, then a wider swiglu-input linear with fewer rows
    cases = [(300, 512, 264, 0), (129, 1024, 136, 1), (300, 512, 264, 0)]
    for (m, k, n, act) in cases:
        width = 2 * k if act else k
        x = torch.randn((m, width), generator=g).to(torch.bfloat16).to(DEV)
        w = torch.randint(-127, 128, (n, k), dtype=torch.int8, generator=g).to(DEV)
        cs = (torch.rand((n,), generator=g) * 0.01 + 1e-4).to(DEV)
        bias = (torch.randn((n,), generator=g) * 0.01).to(torch.bfloat16).to(DEV)
        want = pkg.ops.int8_linear(x, w, cs, bias, input_act="swiglu" if act else None)
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
        st = lib.b2_int8_linear_noalloc(P(x.data_ptr()), act, P(w.data_ptr()), P(cs.data_ptr()),
                                        P(bias.data_ptr()), 1, P(got.data_ptr()), m, n, k, P(stream))
        assert st == 0, lib.b2_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (m, k, n, act)
        if not act:
            # and the CPU oracle's bits (the swiglu case is compared with the scratch entry point
            # only: host and device expf may differ in the last place, as the swiglu tests say)
            oracle = ref.int8_linear(x.cpu(), w.cpu(), cs.cpu(), bias.cpu())
            assert torch.equal(got.cpu().view(torch.int16), oracle.view(torch.int16)), (m, k, n, act)
    pkg.ops.check_device_status()
