"""GPU parity of the multi-pass forms of the tensor-core GEMM (ttb_linear_ex) and of the reference-recipe int8 Linear.

  fp32 as three tf32 products    against the numpy fp32 MatMul restatement (mat_mul.cpp:30-118): fp32-level accuracy
  bf16 hi + lo activation planes against the same product evaluated on the hi + lo sum; two-plane and fp32 outputs
  split-K over a cluster         shapes with M <= 128 and a long K take that route; same oracle, every epilogue
  int8, torch dynamic recipe     weight / activation quantisation bit-exact against the restatement of
                                 qmodeling_bert.py:13-45's torch arithmetic, GEMM + epilogue against qref_linear
"""
import numpy as np
import pytest
import torch

from oracle import restate
from tests.helpers import TORCH_DT, code, dev, host, maxdiff, rng, rounded
from turbotransformers_b200 import _capi

pytestmark = pytest.mark.gpu
EPIS = {"none": 0, "bias": 1, "bias_gelu": 2, "bias_residual": 3, "bias_tanh": 4}


def epilogue_oracle(y, bias, res, epi):
    if epi == "none":
        return y
    if epi == "bias":
        return restate.add_bias(y, bias)
    if epi == "bias_gelu":
        return restate.add_bias_act(y, bias, "gelu")
    if epi == "bias_tanh":
        return restate.add_bias_act(y, bias, "tanh")
    return restate.add_input_bias(y, res, bias)


def prepack(ctx, w_kn, dt):
    K, N = w_kn.shape
    dst = torch.empty((N, K), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("prepack_weight", _capi.F32, dev(w_kn), 0, K, N, code(dt), dst)
    return dst


def split_planes(ctx, t):
    """fp32 device tensor -> (hi, lo) tf32-representable planes through the library's kernel."""
    hi, lo = torch.empty_like(t), torch.empty_like(t)
    ctx.call("split_tf32", t, t.numel(), hi, lo)
    return hi, lo


def test_split_tf32_planes_are_tf32_values_that_add_up(ctx):
    x = torch.randn(1000003, device="cuda") * 3.0
    x = x[:1000000].contiguous()
    hi, lo = split_planes(ctx, x)
    for plane in (hi, lo):
        assert int((plane.view(torch.int32) & 0x1FFF).abs().max().item()) == 0   # 13 low mantissa bits clear
    rel = ((hi + lo - x).abs() / x.abs().clamp_min(1e-30)).max().item()
    assert rel < 2.0 ** -20


@pytest.mark.parametrize("M,N,K", [(128, 768, 768), (128, 768, 3072), (1, 2304, 768), (333, 3072, 768), (2048, 768, 3072),
                                   (4100, 2304, 768), (257, 200, 72)])
@pytest.mark.parametrize("epi", ["none", "bias_gelu", "bias_residual"])
def test_fp32_linear_on_tf32_tensor_cores_has_fp32_accuracy(ctx, M, N, K, epi):
    r = rng(M * 3 + N + K)
    a = r.standard_normal((M, K)).astype(np.float32)
    w = (r.standard_normal((K, N)) * 0.05).astype(np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    res = r.standard_normal((M, N)).astype(np.float32)
    want = epilogue_oracle(restate.mat_mul(a, False, w, False), bias, res, epi)
    A_hi, A_lo = split_planes(ctx, dev(a))
    W_hi, W_lo = split_planes(ctx, prepack(ctx, w, "f32"))
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    ctx.linear_ex(_capi.F32, _capi.F32, A_hi, W_hi, M, N, K, EPIS[epi], out, A2=A_lo, W2=W_lo, bias=dev(bias), residual=dev(res))
    assert ctx.device_status() == _capi.OK
    got = host(out)
    assert np.isfinite(got).all()
    # Three tf32 products drop terms of 2^-21 relative. On top of that the tensor core's fp32 accumulator truncates (it
    # does not round to nearest) at each of its K / 8 accumulation steps, which shows as a shrink of about 1e-8 * K
    # relative: 8e-6 at K = 768, 3e-5 at K = 3072 (a single-pass tf32 GEMM, the reference's tensor-op route, is at 1e-3).
    assert maxdiff(got, want) < max(2e-5, 1.4e-8 * K) * max(1.0, float(np.abs(want).max()))


@pytest.mark.parametrize("M,N,K", [(128, 768, 768), (300, 3072, 768), (2100, 768, 3072), (4100, 2304, 768)])
def test_bf16_two_plane_activations_and_outputs(ctx, M, N, K):
    r = rng(M + N + K)
    a = r.standard_normal((M, K)).astype(np.float32)
    a_hi = rounded(a, "bf16")
    a_lo = rounded(a - a_hi, "bf16")
    w = rounded(r.standard_normal((K, N)).astype(np.float32) * 0.05, "bf16")
    bias = rounded(r.standard_normal(N).astype(np.float32), "bf16")
    Wp = prepack(ctx, w, "bf16")
    y = restate.mat_mul(a_hi + a_lo, False, w, False)
    # (1) bias + GELU written as two bf16 planes: their sum carries 16 significant bits
    want = restate.add_bias_act(y.copy(), bias, "gelu")
    hi = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    lo = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ctx.linear_ex(_capi.BF16, _capi.BF16, dev(a_hi, "bf16"), Wp, M, N, K, EPIS["bias_gelu"], hi, A2=dev(a_lo, "bf16"), bias=dev(bias, "bf16"),
                  out_lo=lo)
    assert ctx.device_status() == _capi.OK
    scale = max(1.0, float(np.abs(want).max()))
    assert maxdiff(host(hi), want) < 2.0 ** -8 * scale + 2e-3                 # the hi plane alone is a bf16 rounding away
    assert maxdiff(host(hi) + host(lo), want) < 2.0 ** -15 * scale + 2e-3     # tanh.approx bounds the rest
    # (2) bias + fp32 residual -> fp32 output (the residual stream of a bf16 model)
    res = r.standard_normal((M, N)).astype(np.float32)
    want2 = restate.add_input_bias(y.copy(), res, bias)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    ctx.linear_ex(_capi.BF16, _capi.F32, dev(a_hi, "bf16"), Wp, M, N, K, EPIS["bias_residual"], out, A2=dev(a_lo, "bf16"), bias=dev(bias),
                  residual=dev(res))
    assert ctx.device_status() == _capi.OK
    assert maxdiff(host(out), want2) < 3e-5 * max(1.0, float(np.abs(want2).max()))


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(128, 768, 3072), (128, 768, 768), (128, 2304, 768), (7, 768, 3072), (100, 1024, 4096), (128, 96, 512)])
@pytest.mark.parametrize("epi", ["none", "bias_gelu", "bias_residual"])
def test_small_problems_split_along_k_over_a_cluster(ctx, dt, M, N, K, epi):
    r = rng(M + N + K + 1)
    a = rounded(r.standard_normal((M, K)).astype(np.float32), dt)
    w = rounded(r.standard_normal((K, N)).astype(np.float32) * 0.05, dt)
    bias = rounded(r.standard_normal(N).astype(np.float32), dt)
    res = rounded(r.standard_normal((M, N)).astype(np.float32), dt)
    want = epilogue_oracle(restate.mat_mul(a, False, w, False), bias, res, epi)
    Wp = prepack(ctx, w, dt)
    outs = []
    for _ in range(2):  # twice: the result must not depend on which CTA of the cluster finishes first
        out = torch.full((M, N), float("nan"), dtype=TORCH_DT[dt], device="cuda")
        ctx.call("linear", code(dt), dev(a, dt), K, Wp, dev(bias, dt), dev(res, dt), N, M, N, K, EPIS[epi], out, N)
        outs.append(out)
    assert ctx.device_status() == _capi.OK
    assert torch.equal(outs[0], outs[1])
    scale = max(1.0, float(np.abs(want).max()))
    assert maxdiff(host(outs[0]), want) < (2.0 ** -10 if dt == "f16" else 2.0 ** -7) * scale + 2e-3


@pytest.mark.parametrize("M,N,K", [(128, 3072, 768), (128, 768, 3072), (2048, 3072, 768), (77, 768, 768), (2500, 768, 3072)])
@pytest.mark.parametrize("epi", ["none", "bias_gelu", "bias_residual"])
def test_int8_reference_recipe_linear(ctx, M, N, K, epi):
    r = rng(M + 2 * N)
    x = rounded(r.standard_normal((M, K)).astype(np.float32) + 0.3, "f16")
    x[0, 0] = 6.5   # an outlier sets the range, as in real activations
    w = r.standard_normal((K, N)).astype(np.float32) * 0.02
    bias = rounded(r.standard_normal(N).astype(np.float32) * 0.1, "f16")
    res = rounded(r.standard_normal((M, N)).astype(np.float32), "f16")
    # weights: bit-exact against the restatement of torch's observer + quantiser
    wq, ws = restate.qref_quantize_weight(w)
    Wq = torch.empty((N, K), dtype=torch.int8, device="cuda")
    Ws = torch.zeros(1, dtype=torch.float32, device="cuda")
    Cs = torch.empty(N, dtype=torch.int32, device="cuda")
    ctx.call("prepack_weight_int8_affine", _capi.F32, dev(w), 0, K, N, Wq, Ws, Cs)
    assert float(Ws.item()) == float(ws)
    assert (Wq.cpu().numpy() == wq.T).all()
    assert (Cs.cpu().numpy() == wq.astype(np.int64).sum(0)).all()
    # activations: per-tensor affine, 7 bits
    xq, xs, zp = restate.qref_quantize_activations(x)
    Xq = torch.empty((M, K), dtype=torch.int8, device="cuda")
    Qp = torch.zeros(4, dtype=torch.float32, device="cuda")
    ctx.call("quantize_tensor_affine", _capi.F16, dev(x, "f16"), M, K, Xq, Qp)
    qp = Qp.cpu().numpy()
    assert float(qp[0]) == float(xs) and int(qp[1]) == zp
    assert (Xq.cpu().numpy().astype(np.int32) == xq).all()
    y = epilogue_oracle(restate.qref_linear(x, wq, ws), bias, res, epi)
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    ctx.call("linear_int8_affine", _capi.F16, Xq, Qp, Wq, Ws, Cs, dev(bias, "f16"), dev(res, "f16"), N, M, N, K, EPIS[epi], out, N)
    assert ctx.device_status() == _capi.OK
    scale = max(1.0, float(np.abs(y).max()))
    assert maxdiff(host(out), y) < 2.0 ** -10 * scale + 2e-3


def test_linear_ex_rejects_bad_arguments(ctx):
    import ctypes as C
    a = torch.zeros(8, 16, device="cuda", dtype=torch.float32)
    h = torch.zeros(8, 16, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(_capi.TTBError):   # a second weight plane without a second activation plane
        ctx.linear_ex(_capi.F32, _capi.F32, a, a, 8, 8, 16, 0, a, W2=a)
    with pytest.raises(_capi.TTBError):   # second output plane on an fp32 output
        ctx.linear_ex(_capi.BF16, _capi.F32, h, h, 8, 8, 16, 0, a, out_lo=a)
    with pytest.raises(_capi.TTBError):   # fp32 operands, 16-bit output
        ctx.linear_ex(_capi.F32, _capi.F16, a, a, 8, 8, 16, 0, h)
    assert _capi.lib().ttb_linear_ex(ctx.h, None) == _capi.ERR_INVALID


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(1024, 768, 768), (4100, 768, 3072), (18424, 768, 768), (2049, 1024, 1024), (1500, 256, 512), (3000, 512, 64),
                                   (300, 768, 768), (2048, 640, 768)])
def test_linear_with_layernorm_epilogue(ctx, dt, M, N, K, monkeypatch):
    """out = LayerNorm(A . W^T + bias + residual): the one-kernel form (row sums exchanged between the CTAs of a row block,
    switched on for every K here) against the two kernels in sequence and against the numpy restatement; shapes outside
    its range take the two-kernel route inside the same call (the last two)."""
    monkeypatch.setenv("TTB_GEMM_LN", "2")
    r = rng(M + N + K)
    a = rounded(r.standard_normal((M, K)).astype(np.float32), dt)
    w = rounded(r.standard_normal((K, N)).astype(np.float32) * 0.05, dt)
    bias = rounded(r.standard_normal(N).astype(np.float32), dt)
    res = rounded(r.standard_normal((M, N)).astype(np.float32) * 2.0, dt)
    gamma = rounded(1.0 + 0.2 * r.standard_normal(N).astype(np.float32), dt)
    beta = rounded(0.3 * r.standard_normal(N).astype(np.float32), dt)
    Wp = prepack(ctx, w, dt)
    A, B, R, G, Be = dev(a, dt), dev(bias, dt), dev(res, dt), dev(gamma, dt), dev(beta, dt)
    two = torch.empty((M, N), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("linear", code(dt), A, K, Wp, B, R, N, M, N, K, EPIS["bias_residual"], two, N)
    summed = two.clone()
    ctx.call("layernorm", code(dt), two, two, G, Be, M, N, 1e-12)
    outs = []
    for _ in range(2):
        out = torch.full((M + 1, N), float("nan"), dtype=TORCH_DT[dt], device="cuda")
        ctx.call("linear_layernorm", code(dt), A, K, Wp, B, R, N, G, Be, 1e-12, M, N, K, out, N)
        outs.append(out)
    assert ctx.device_status() == _capi.OK
    assert torch.isnan(outs[0][M]).all()               # nothing written behind the last row
    assert torch.equal(outs[0][:M], outs[1][:M])       # deterministic
    ulp = 2.0 ** -10 if dt == "f16" else 2.0 ** -7
    scale = max(1.0, float(two.float().abs().max().item()))
    # same rounded sum, same formula, another summation order of the row statistics: a last-place difference at most
    assert maxdiff(host(outs[0][:M]), host(two)) <= 2 * ulp * scale
    want = restate.layer_norm(host(summed), gamma, beta, 1e-12)
    assert maxdiff(host(outs[0][:M]), want) < 4 * ulp * scale
