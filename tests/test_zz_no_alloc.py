"""GPU: the allocation-free int8 Linear (ttb_linear_int8_dynamic_noalloc) against the regular two-call path.

Some callers of this library cannot allocate device memory at the point where they need a Linear: their own
arena owns the whole GPU, they are inside a region where the CUDA allocator must not run, or they reach the
library through an FFI that only passes input and output pointers. For them the scratch of the int8 path (the
quantised activations and their row scales) sits in a fixed array inside the library. This test calls the new
entry point twice in a row with different shapes, so the second call sees the first one's leftovers in the
shared array, and requires bit-identical results to ttb_quantize_rows_int8 + ttb_linear_int8 with caller-owned
scratch (the same kernels run, so no tolerance is needed). It also checks the size limit is refused cleanly.
This file sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import pytest
import torch

from turbotransformers_b200 import _capi

pytestmark = pytest.mark.gpu


def _reference_path(ctx, x, Wq, Ws, bias, res, epi):
    M, K = x.shape
    N = Wq.shape[0]
    xq = torch.empty((M, K), dtype=torch.int8, device="cuda")
    xs = torch.empty(M, dtype=torch.float32, device="cuda")
    out = torch.empty((M, N), dtype=x.dtype, device="cuda")
    ctx.call("quantize_rows_int8", _capi.dtype_code(x.dtype), x, M, K, xq, xs)
    ctx.call("linear_int8", _capi.dtype_code(x.dtype), xq, xs, Wq, Ws, bias, res, N, M, N, K, epi, out, N)
    return out


def _noalloc_path(ctx, x, Wq, Ws, bias, res, epi):
    M, K = x.shape
    N = Wq.shape[0]
    out = torch.full((M, N), float("nan"), dtype=x.dtype, device="cuda")
    ctx.call("linear_int8_dynamic_noalloc", _capi.dtype_code(x.dtype), x, Wq, Ws, bias, res, N, M, N, K, epi, out, N)
    return out


def test_noalloc_int8_linear_matches_two_call_path_on_consecutive_calls(ctx):
    g = torch.Generator(device="cuda").manual_seed(0)
    cases = [(torch.float16, 2048, 3072, 768, _capi.EPI_BIAS_GELU),   # first call fills most of the scratch
             (torch.float16, 77, 768, 3072, _capi.EPI_BIAS_RESIDUAL),  # second call: smaller, different K, sees leftovers
             (torch.bfloat16, 300, 2304, 768, _capi.EPI_BIAS)]
    for dt, M, N, K, epi in cases:
        x = torch.randn(M, K, device="cuda", dtype=dt, generator=g)
        Wq = torch.randint(-127, 128, (N, K), device="cuda", dtype=torch.int8, generator=g)
        Ws = torch.full((1,), 0.0007, device="cuda", dtype=torch.float32)
        bias = torch.randn(N, device="cuda", dtype=dt, generator=g)
        res = torch.randn(M, N, device="cuda", dtype=dt, generator=g)
        want = _reference_path(ctx, x, Wq, Ws, bias, res, epi)
        got = _noalloc_path(ctx, x, Wq, Ws, bias, res, epi)
        assert ctx.device_status() == _capi.OK
        assert torch.isfinite(got.float()).all()
        assert torch.equal(got, want)
        # and once more right away: same inputs, same shared array, same answer
        assert torch.equal(_noalloc_path(ctx, x, Wq, Ws, bias, res, epi), want)


def test_noalloc_rejects_problems_beyond_its_scratch(ctx):
    lib = _capi.lib()
    x = torch.zeros(8, 16, device="cuda", dtype=torch.float16)
    P = lambda t: C.c_void_p(t.data_ptr())
    before = ctx.launches()
    # M*K beyond 8 Mi elements, and M beyond 65536 rows: refused before anything is launched
    assert lib.ttb_linear_int8_dynamic_noalloc(ctx.h, _capi.F16, P(x), P(x), P(x), None, None, 0, 4096, 768, 4096, 0, P(x), 768) \
        == _capi.ERR_INVALID
    assert b"exceeds the built-in scratch" in lib.ttb_last_error(ctx.h)
    assert lib.ttb_linear_int8_dynamic_noalloc(ctx.h, _capi.F16, P(x), P(x), P(x), None, None, 0, 70000, 768, 16, 0, P(x), 768) \
        == _capi.ERR_INVALID
    assert ctx.launches() == before
    # every other invalid argument is also refused before the quantising kernel could overwrite the shared array:
    # K not a multiple of 16, an fp32 activation dtype, an epilogue without its bias, an output pitch below N, a null weight
    for args in ((_capi.F16, P(x), P(x), P(x), None, None, 0, 8, 8, 24, 0, P(x), 8),
                 (_capi.F32, P(x), P(x), P(x), None, None, 0, 8, 8, 16, 0, P(x), 8),
                 (_capi.F16, P(x), P(x), P(x), None, None, 0, 8, 8, 16, _capi.EPI_BIAS, P(x), 8),
                 (_capi.F16, P(x), P(x), P(x), None, None, 0, 8, 16, 16, 0, P(x), 8),
                 (_capi.F16, P(x), None, P(x), None, None, 0, 8, 8, 16, 0, P(x), 8)):
        assert lib.ttb_linear_int8_dynamic_noalloc(ctx.h, *args) == _capi.ERR_INVALID
    assert ctx.launches() == before
    assert lib.ttb_linear_int8_dynamic_noalloc(ctx.h, _capi.F16, P(x), P(x), P(x), None, None, 0, 0, 768, 16, 0, P(x), 768) == _capi.OK
