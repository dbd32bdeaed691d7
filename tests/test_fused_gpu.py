"""GPU parity of the fused tensor-core entry points (ttb_linear, ttb_linear_int8, ttb_attention_fwd)
against the numpy restatement of the reference's unfused CPU sequence, on inputs rounded to the storage type.

fp16/bf16 tolerance: the accumulator is fp32, so the error is the output rounding (2^-11 / 2^-8 relative)
plus tanh.approx in the GELU epilogue; int8: the int32 accumulator is exact, so only the fp16 rounding of
the dequantised result remains.
"""
import math

import numpy as np
import pytest
import torch

from oracle import restate
from tests.helpers import TORCH_DT, code, dev, host, maxdiff, rng, rounded
from turbotransformers_b200 import _capi

pytestmark = pytest.mark.gpu

EPIS = {"none": 0, "bias": 1, "bias_gelu": 2, "bias_residual": 3, "bias_tanh": 4}


def prepack(ctx, w_kn, dt):
    """[K,N] fp32 numpy -> device [N,K] in dt through the library's own re-layout kernel."""
    K, N = w_kn.shape
    dst = torch.empty((N, K), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("prepack_weight", _capi.F32, dev(w_kn), 0, K, N, code(dt), dst)
    return dst


def linear_oracle(a, w_kn, bias, res, epi):
    """The reference's unfused sequence: MatMul (mat_mul.cpp:30-118) then the elementwise kernel."""
    y = restate.mat_mul(a, False, w_kn, False)
    if epi == "none":
        return y
    if epi == "bias":
        return restate.add_bias(y, bias)
    if epi == "bias_gelu":
        return restate.add_bias_act(y, bias, "gelu")
    if epi == "bias_tanh":
        return restate.add_bias_act(y, bias, "tanh")
    return restate.add_input_bias(y, res, bias)


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(128, 768, 768), (128, 2304, 768), (128, 3072, 768), (128, 768, 3072),
                                   (1, 768, 768), (5, 768, 3072), (200, 2304, 768), (333, 768, 3072),
                                   (1000, 3072, 768), (4096, 1024, 1024), (257, 200, 72), (130, 50264, 768),
                                   (2048, 3072, 768), (1500, 5120, 200)])  # the last three run on CTA pairs
@pytest.mark.parametrize("epi", ["bias", "bias_gelu", "bias_residual"])
def test_linear_matches_unfused_reference(ctx, dt, M, N, K, epi):
    if N > 10000 and epi != "bias":
        pytest.skip("vocabulary-sized N is only used with the plain bias epilogue")
    r = rng(M + N + K)
    a = rounded(r.standard_normal((M, K)).astype(np.float32), dt)
    w = rounded(r.standard_normal((K, N)).astype(np.float32) * 0.05, dt)
    bias = rounded(r.standard_normal(N).astype(np.float32), dt)
    res = rounded(r.standard_normal((M, N)).astype(np.float32), dt)
    want = linear_oracle(a, w, bias, res, epi)
    Wp = prepack(ctx, w, dt)
    assert maxdiff(host(Wp), w.T) == 0.0
    out = torch.full((M, N), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("linear", code(dt), dev(a, dt), K, Wp, dev(bias, dt), dev(res, dt), N, M, N, K, EPIS[epi], out, N)
    assert ctx.device_status() == _capi.OK
    got = host(out)
    assert np.isfinite(got).all()
    scale = max(1.0, float(np.abs(want).max()))
    tol = (2.0 ** -10 if dt == "f16" else 2.0 ** -7) * scale + 2e-3
    assert maxdiff(got, want) < tol


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_linear_plain_and_tanh_epilogues_and_strided_io(ctx, dt):
    r = rng(77)
    M, N, K = 300, 768, 768
    a_full = rounded(r.standard_normal((M, 3 * K)).astype(np.float32), dt)  # A is a column slice: lda = 3K
    a = a_full[:, K:2 * K]
    w = rounded(r.standard_normal((K, N)).astype(np.float32) * 0.05, dt)
    bias = rounded(r.standard_normal(N).astype(np.float32), dt)
    Wp = prepack(ctx, w, dt)
    A = dev(a_full, dt)
    out = torch.zeros((M, 2 * N), dtype=TORCH_DT[dt], device="cuda")  # written into the right half: ldo = 2N
    es = out.element_size()
    import ctypes as C
    _capi.lib().ttb_linear(ctx.h, code(dt), C.c_void_p(A.data_ptr() + K * es), 3 * K, C.c_void_p(Wp.data_ptr()), None, None, 0,
                           M, N, K, EPIS["none"], C.c_void_p(out.data_ptr() + N * es), 2 * N)
    got = host(out)
    assert maxdiff(got[:, :N], 0) == 0.0
    assert maxdiff(got[:, N:], restate.mat_mul(a, False, w, False)) < (0.02 if dt == "f16" else 0.12)
    out2 = torch.zeros((M, N), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("linear", code(dt), dev(a, dt), K, Wp, dev(bias, dt), None, 0, M, N, K, EPIS["bias_tanh"], out2, N)
    assert maxdiff(host(out2), linear_oracle(a, w, bias, None, "bias_tanh")) < (4e-3 if dt == "f16" else 2e-2)


@pytest.mark.parametrize("M,N,K", [(300, 1001, 256), (2100, 5003, 768)])  # the second runs on CTA pairs
def test_linear_ragged_width_into_padded_rows_then_compacted(ctx, M, N, K):
    # how a 50257-wide vocabulary projection runs: no bias, rows padded to a multiple of 8 elements, then ttb_copy_2d
    dt = "f16"
    r = rng(N)
    a = rounded(r.standard_normal((M, K)).astype(np.float32), dt)
    w = rounded(r.standard_normal((K, N)).astype(np.float32) * 0.05, dt)
    Wp = prepack(ctx, w, dt)
    Np = (N + 7) // 8 * 8
    padded = torch.full((M, Np), 7.0, dtype=torch.float16, device="cuda")
    want = restate.mat_mul(a, False, w, False)
    tol = 2.0 ** -10 * max(1.0, float(np.abs(want).max())) + 2e-3
    ctx.call("linear", code(dt), dev(a, dt), K, Wp, None, None, 0, M, N, K, EPIS["none"], padded, Np)
    got = host(padded)
    assert maxdiff(got[:, N:], 7.0) == 0.0  # without the flag the padding columns are not written
    assert maxdiff(got[:, :N], want) < tol
    ctx.call("linear", code(dt), dev(a, dt), K, Wp, None, None, 0, M, N, K, EPIS["none"] | 0x100, padded, Np)  # padding declared scratch
    assert ctx.device_status() == _capi.OK
    got = host(padded)
    assert maxdiff(got[:, :N], want) < 2.0 ** -10 * max(1.0, float(np.abs(want).max())) + 2e-3
    out = torch.empty((M, N), dtype=torch.float16, device="cuda")
    ctx.call("copy_2d", out, N * 2, padded, Np * 2, N * 2, M)
    assert maxdiff(host(out), got[:, :N]) == 0.0


def test_linear_weight_given_as_out_in(ctx):
    # is_trans_weight=True in the reference: the weight arrives as [N,K] and is only converted
    r = rng(5)
    K, N, M = 768, 768, 64
    w_nk = r.standard_normal((N, K)).astype(np.float32) * 0.05
    dst = torch.empty((N, K), dtype=torch.float16, device="cuda")
    ctx.call("prepack_weight", _capi.F32, dev(w_nk), 1, K, N, _capi.F16, dst)
    assert maxdiff(host(dst), rounded(w_nk, "f16")) == 0.0


def test_linear_large_m_roundtrip_property(ctx):
    # full benchmark-size M: identity weights must return the input exactly (checks every tile and row)
    M, K = 18424, 768
    a = torch.randn(M, K, device="cuda", dtype=torch.float16)
    eye = torch.eye(K, device="cuda", dtype=torch.float16)
    zero = torch.zeros(K, device="cuda", dtype=torch.float16)
    out = torch.empty_like(a)
    ctx.call("linear", _capi.F16, a, K, eye, zero, None, 0, M, K, K, EPIS["bias"], out, K)
    assert ctx.device_status() == _capi.OK
    assert torch.equal(out, a)
    # linearity in A: f(2a) == 2 f(a) exactly in binary floating point
    w = torch.randn(K, K, device="cuda", dtype=torch.float16) * 0.05
    o1, o2 = torch.empty_like(a), torch.empty_like(a)
    ctx.call("linear", _capi.F16, a, K, w, zero, None, 0, M, K, K, EPIS["none"], o1, K)
    ctx.call("linear", _capi.F16, a * 2, K, w, zero, None, 0, M, K, K, EPIS["none"], o2, K)
    normal = o1.abs() >= 2.0 ** -13  # a subnormal fp16 result has an absolute rounding step, so only normal ones scale exactly
    assert torch.equal(o2[normal], (o1 * 2)[normal])
    assert (o2.float() - 2 * o1.float()).abs().max().item() <= 2.0 ** -23
    ref = (a[:512].float() @ w.float().T)
    assert (o1[:512].float() - ref).abs().max().item() < 0.02


def test_linear_rejects_bad_arguments(ctx):
    lib = _capi.lib()
    a = torch.zeros(8, 12, device="cuda", dtype=torch.float16)
    import ctypes as C
    P = lambda t: C.c_void_p(t.data_ptr())
    assert lib.ttb_linear(ctx.h, _capi.F16, P(a), 12, P(a), None, None, 0, 8, 8, 12, 0, P(a), 8) == _capi.ERR_INVALID  # K % 8
    assert lib.ttb_linear(ctx.h, _capi.F32, P(a), 16, P(a), None, None, 0, 8, 8, 16, 0, P(a), 8) == _capi.ERR_INVALID  # dtype
    assert lib.ttb_linear(ctx.h, _capi.F16, P(a), 16, P(a), None, None, 0, 8, 8, 16, 1, P(a), 8) == _capi.ERR_INVALID  # no bias
    assert lib.ttb_linear(ctx.h, _capi.F16, P(a), 16, P(a), None, None, 0, 0, 8, 16, 0, P(a), 8) == _capi.OK  # empty


# ------------------------------------------------------------------------------------------------ int8
@pytest.mark.parametrize("M,N,K", [(128, 3072, 768), (128, 768, 3072), (16 * 128, 2304, 768), (77, 768, 768), (2048, 3072, 768)])
@pytest.mark.parametrize("epi", ["bias", "bias_gelu", "bias_residual"])
def test_int8_linear_matches_integer_oracle(ctx, M, N, K, epi):
    r = rng(M + N)
    x = rounded(r.standard_normal((M, K)).astype(np.float32), "f16")
    w = r.standard_normal((K, N)).astype(np.float32) * 0.02
    bias = rounded(r.standard_normal(N).astype(np.float32) * 0.1, "f16")
    res = rounded(r.standard_normal((M, N)).astype(np.float32), "f16")
    wq, ws = restate.q_quantize_weight(w)
    # weight quantisation on the device must agree with the oracle bit for bit
    Wq = torch.empty((N, K), dtype=torch.int8, device="cuda")
    Ws = torch.zeros(1, dtype=torch.float32, device="cuda")
    ctx.call("prepack_weight_int8", _capi.F32, dev(w), 0, K, N, Wq, Ws)
    assert abs(float(Ws.item()) - float(ws)) <= 1e-9 + 1e-6 * float(ws)
    assert (Wq.cpu().numpy() == wq.T).all()
    # activation quantisation: bit-exact too
    Xq = torch.empty((M, K), dtype=torch.int8, device="cuda")
    Xs = torch.empty(M, dtype=torch.float32, device="cuda")
    ctx.call("quantize_rows_int8", _capi.F16, dev(x, "f16"), M, K, Xq, Xs)
    xq, xs = restate.q_quantize_rows(x)
    assert (Xq.cpu().numpy() == xq).all() and maxdiff(host(Xs), xs.reshape(-1)) < 1e-7
    y = restate.q_linear(x, wq, ws, bias)
    if epi == "bias_gelu":
        y = restate.gelu_tanh(y)
    elif epi == "bias_residual":
        y = y + res
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device="cuda")
    ctx.call("linear_int8", _capi.F16, Xq, Xs, Wq, Ws, dev(bias, "f16"), dev(res, "f16"), N, M, N, K, EPIS[epi], out, N)
    assert ctx.device_status() == _capi.OK
    scale = max(1.0, float(np.abs(y).max()))
    assert maxdiff(host(out), y) < 2.0 ** -10 * scale + 2e-3


# ------------------------------------------------------------------------------------------- attention
def attention_oracle(qkv, lens, heads, mask=None, causal=False):
    """Per sequence: BatchMatMul(q,k^T,1/sqrt(d)) -> ApplyMaskAndSoftmax -> BatchMatMul(p,v) -> TransposeForScore
    (multi_headed_attention.cpp:320-354) on the packed [T,3H] projection."""
    H = qkv.shape[1] // 3
    d = H // heads
    outs, s = [], 0
    for b, n in enumerate(lens):
        x = qkv[s:s + n].reshape(1, n, 3, heads, d)
        q, k, v = (np.ascontiguousarray(np.transpose(x[:, :, i], (0, 2, 1, 3))) for i in range(3))
        score = restate.batch_mat_mul(q, False, k, True, 1.0 / math.sqrt(d))
        m = None
        if mask is not None:
            m = mask[b:b + 1, ..., :n] if mask.ndim == 2 else mask[b:b + 1, :n, :n]
        if causal:
            cm = restate.causal_mask(1, n, -1e9)
            m = cm if m is None else cm + (m.reshape(1, 1, n) if m.ndim == 2 else m)
        prob = restate.apply_mask_and_softmax(score, m, 1.0)
        outs.append(restate.transpose_for_score(restate.batch_mat_mul(prob, False, v, False))[0])
        s += n
    return np.concatenate(outs)


@pytest.mark.parametrize("kernel", ["auto", "tensor_memory", "mma_sync"])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("lens,heads", [([128], 12), ([4, 1], 12), ([9, 7, 13], 4), ([37, 5, 128, 64], 12),
                                        ([511, 8, 300, 65, 64, 63, 1], 12), ([512], 16), ([512, 512, 480], 2)])
def test_attention_varlen(ctx, dt, lens, heads, kernel, monkeypatch):
    # both attention kernels are checked on every shape; "auto" is what callers get
    if kernel != "auto":
        monkeypatch.setenv("TTB_ATTN_TC", "2" if kernel == "tensor_memory" else "0")
    r = rng(sum(lens))
    H, T = heads * 64, sum(lens)
    qkv = rounded(r.standard_normal((T, 3 * H)).astype(np.float32), dt)
    want = attention_oracle(qkv, lens, heads)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32).cuda()
    out = torch.full((T, H), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("attention_fwd", code(dt), dev(qkv, dt), T, cu, len(lens), max(lens), heads, 64, None, 0, 0, 0, 0.125, out)
    got = host(out)
    assert np.isfinite(got).all()
    assert maxdiff(got, want) < (4e-3 if dt == "f16" else 3e-2)


@pytest.mark.parametrize("kernel", ["auto", "tensor_memory", "mma_sync"])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("lens,heads,pitch,causal", [([512, 300, 129, 8, 477, 64, 390, 511, 1, 256, 500, 128], 12, 512, False),
                                                     ([200, 131, 77], 4, 203, False),     # odd pitch: the scalar mask loads
                                                     ([384, 250, 512], 4, 512, True),     # padding mask on top of the causal flag
                                                     ([1100, 640], 2, 1100, False)])
def test_attention_with_a_per_key_mask(ctx, dt, lens, heads, pitch, causal, kernel, monkeypatch):
    """The encoder's padding mask ([B, Lk] additive, one row of keys per sequence) on every kernel: 0 / -10000 entries
    as PrepareBertMasks makes them plus a few graded ones, ragged lengths, key tiles that end inside a tile."""
    if kernel != "auto":
        monkeypatch.setenv("TTB_ATTN_TC", "2" if kernel == "tensor_memory" else "0")
    r = rng(sum(lens) + pitch)
    H, T, B = heads * 64, sum(lens), len(lens)
    qkv = rounded(r.standard_normal((T, 3 * H)).astype(np.float32), dt)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32).cuda()
    mask = np.where(r.random((B, pitch)) < 0.3, -10000.0, 0.0).astype(np.float32)
    mask += np.where(r.random((B, pitch)) < 0.1, -3.0 * r.random((B, pitch)), 0.0).astype(np.float32)
    mask[:, 0] = 0   # every query keeps at least one key
    mask[0, :] = 0   # one sequence without padding
    out = torch.full((T, H), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("attention_fwd", code(dt), dev(qkv, dt), T, cu, B, max(lens), heads, 64, dev(mask), pitch, 0, int(causal), 0.125, out)
    assert ctx.device_status() == _capi.OK
    got = host(out)
    assert np.isfinite(got).all()
    assert maxdiff(got, attention_oracle(qkv, lens, heads, mask, causal=causal)) < (4e-3 if dt == "f16" else 3e-2)


@pytest.mark.parametrize("kernel", ["auto", "tensor_memory", "mma_sync"])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("value", [-10000.0, -3.0e38])
def test_attention_with_a_padding_mask(ctx, dt, kernel, value, monkeypatch):
    """A padded batch the way HuggingFace callers pass it: every sequence has the full length and a suffix of its keys
    masked out (whole key tiles among them, which the kernels skip), kept lengths from one key to all of them."""
    if kernel != "auto":
        monkeypatch.setenv("TTB_ATTN_TC", "2" if kernel == "tensor_memory" else "0")
    r = rng(77)
    B, L, heads = 9, 512, 4
    keep = [512, 1, 127, 128, 129, 300, 384, 385, 64]
    H, T = heads * 64, B * L
    qkv = rounded(r.standard_normal((T, 3 * H)).astype(np.float32), dt)
    cu = torch.tensor(np.arange(B + 1) * L, dtype=torch.int32).cuda()
    mask = np.zeros((B, L), np.float32)
    for b, n in enumerate(keep):
        mask[b, n:] = value
    out = torch.full((T, H), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("attention_fwd", code(dt), dev(qkv, dt), T, cu, B, L, heads, 64, dev(mask), L, 0, 0, 0.125, out)
    assert ctx.device_status() == _capi.OK
    got = host(out)
    assert np.isfinite(got).all()
    oracle_mask = np.maximum(mask, -1.0e9)   # the same softmax without overflowing the float32 restatement
    assert maxdiff(got, attention_oracle(qkv, [L] * B, heads, oracle_mask)) < (4e-3 if dt == "f16" else 3e-2)


@pytest.mark.parametrize("kernel", ["tensor_memory", "mma_sync"])
@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_attention_masks_and_causal(ctx, dt, kernel, monkeypatch):
    # per-key masks are an operand of both kernels; masks with a row per query always take mma.sync
    monkeypatch.setenv("TTB_ATTN_TC", "2" if kernel == "tensor_memory" else "0")
    r = rng(21)
    lens, heads = [70, 33, 128], 4
    H, T, B, maxL = heads * 64, sum(lens), len(lens), max(lens)
    qkv = rounded(r.standard_normal((T, 3 * H)).astype(np.float32), dt)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32).cuda()
    Q = dev(qkv, dt)
    tol = 4e-3 if dt == "f16" else 3e-2
    # per-key additive mask [B, maxL] (BERT's extended mask: 0 / -10000)
    m2 = np.where(r.random((B, maxL)) < 0.25, -10000.0, 0.0).astype(np.float32)
    m2[:, 0] = 0
    out = torch.zeros((T, H), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("attention_fwd", code(dt), Q, T, cu, B, maxL, heads, 64, dev(m2), maxL, 0, 0, 0.125, out)
    assert maxdiff(host(out), attention_oracle(qkv, lens, heads, m2)) < tol
    # per-query mask [B, maxL, maxL]
    m3 = np.where(r.random((B, maxL, maxL)) < 0.25, -1e9, 0.0).astype(np.float32)
    m3[:, :, 0] = 0
    ctx.call("attention_fwd", code(dt), Q, T, cu, B, maxL, heads, 64, dev(m3), maxL * maxL, maxL, 0, 0.125, out)
    assert maxdiff(host(out), attention_oracle(qkv, lens, heads, m3)) < tol
    # causal flag == explicit lower-triangular mask
    ctx.call("attention_fwd", code(dt), Q, T, cu, B, maxL, heads, 64, None, 0, 0, 1, 0.125, out)
    assert maxdiff(host(out), attention_oracle(qkv, lens, heads, None, causal=True)) < tol


def test_attention_permutation_property_at_benchmark_size(ctx):
    # 64 sequences with lengths in [8,512]: reversing the batch order must permute the output rows, bit for bit
    from turbotransformers_b200 import synthetic
    lens = synthetic.varlen_lengths(64, 8, 512, 0)
    heads, H, T = 12, 768, sum(lens)
    qkv = torch.randn(T, 3 * H, device="cuda", dtype=torch.float16)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32).cuda()
    out = torch.empty(T, H, device="cuda", dtype=torch.float16)
    ctx.call("attention_fwd", _capi.F16, qkv, T, cu, 64, max(lens), heads, 64, None, 0, 0, 0, 0.125, out)
    starts = np.concatenate([[0], np.cumsum(lens)])
    order = list(range(63, -1, -1))
    qkv_r = torch.cat([qkv[starts[b]:starts[b + 1]] for b in order])
    lens_r = [lens[b] for b in order]
    cu_r = torch.tensor(np.concatenate([[0], np.cumsum(lens_r)]), dtype=torch.int32).cuda()
    out_r = torch.empty_like(out)
    ctx.call("attention_fwd", _capi.F16, qkv_r, T, cu_r, 64, max(lens), heads, 64, None, 0, 0, 0, 0.125, out_r)
    want = torch.cat([out[starts[b]:starts[b + 1]] for b in order])
    assert torch.equal(out_r, want)
    # rows of a softmax-weighted average stay inside the value range of their sequence
    v = qkv[:, 2 * H:].float()
    assert out.float().abs().max() <= v.abs().max() + 1e-3


def test_attention_kernels_agree_on_repeated_launches_at_benchmark_size(ctx, monkeypatch):
    # The tensor-memory kernel hands buffers between its warps through barriers; a missing one shows up as an
    # intermittent mismatch at full size, not on small cases. 25 launches against the mma.sync kernel's output.
    from turbotransformers_b200 import synthetic
    lens = synthetic.varlen_lengths(64, 8, 512, 0)
    heads, H, T = 12, 768, sum(lens)
    qkv = torch.randn(T, 3 * H, device="cuda", dtype=torch.float16)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device="cuda")
    out = torch.empty(T, H, device="cuda", dtype=torch.float16)

    def run():
        ctx.call("attention_fwd", _capi.F16, qkv, T, cu, len(lens), max(lens), heads, 64, None, 0, 0, 0, 0.125, out)
        torch.cuda.synchronize()
        assert ctx.device_status() == _capi.OK

    monkeypatch.setenv("TTB_ATTN_TC", "0")
    run()
    ref = out.clone()
    monkeypatch.setenv("TTB_ATTN_TC", "2")
    first = None
    for _ in range(25):
        out.zero_()
        run()
        assert (out.float() - ref.float()).abs().max().item() < 4e-3
        if first is None:
            first = out.clone()
        assert torch.equal(out, first)  # and bit-identical from launch to launch



@pytest.mark.parametrize("kernel", ["tensor_memory", "mma_sync"])
@pytest.mark.parametrize("case", ["empty_sequences", "many_sequences", "long_sequence", "long_causal", "beyond_schedule_tables"])
def test_attention_edge_batches(ctx, kernel, case, monkeypatch):
    """Shapes at the edges of the tensor-memory kernel's schedule: zero-length sequences inside a batch, more sequences than its
    length ranking handles (256) and than its tables hold (512: the dispatcher must fall back), and sequences of many key tiles."""
    monkeypatch.setenv("TTB_ATTN_TC", "2" if kernel == "tensor_memory" else "0")
    r = rng(len(case))
    causal = case == "long_causal"
    if case == "empty_sequences":
        lens, heads = [0, 37, 0, 0, 130, 1, 0], 2
    elif case == "many_sequences":
        lens, heads = [int(v) for v in r.integers(1, 40, 300)], 1
    elif case == "beyond_schedule_tables":
        lens, heads = [int(v) for v in r.integers(1, 12, 600)], 1
    else:
        lens, heads = [1500, 700], 1
    H, T = heads * 64, sum(lens)
    qkv = rounded(r.standard_normal((T, 3 * H)).astype(np.float32), "f16")
    want = attention_oracle(qkv, [n for n in lens if n > 0], heads, causal=causal)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32).cuda()
    out = torch.full((T, H), float("nan"), dtype=torch.float16, device="cuda")
    ctx.call("attention_fwd", _capi.F16, dev(qkv, "f16"), T, cu, len(lens), max(lens), heads, 64, None, 0, 0, int(causal), 0.125, out)
    assert ctx.device_status() == _capi.OK
    got = host(out)
    assert np.isfinite(got).all()
    assert maxdiff(got, want) < 4e-3


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("M,N", [(300, 768), (1, 768), (4097, 1024), (50, 256), (33, 3072), (7, 100)])
def test_layernorm_with_int8_output_equals_the_two_kernels_in_sequence(ctx, dt, M, N):
    r = rng(M + N)
    x = dev(r.standard_normal((M, N)).astype(np.float32) * 2.0 + 0.5, dt)
    g = dev(1.0 + 0.1 * r.standard_normal(N).astype(np.float32), dt)
    b = dev(0.1 * r.standard_normal(N).astype(np.float32), dt)
    want = torch.empty_like(x)
    ctx.call("layernorm", code(dt), x, want, g, b, M, N, 1e-12)
    want_q = torch.empty((M, N), dtype=torch.int8, device="cuda")
    want_s = torch.empty(M, dtype=torch.float32, device="cuda")
    ctx.call("quantize_rows_int8", code(dt), want, M, N, want_q, want_s)
    out = x.clone()
    q = torch.full((M, N), 99, dtype=torch.int8, device="cuda")
    s = torch.full((M,), -1.0, dtype=torch.float32, device="cuda")
    ctx.call("layernorm_quant_int8", code(dt), out, out, q, s, g, b, M, N, 1e-12)   # in place
    assert ctx.device_status() == _capi.OK
    assert torch.equal(out, want) and torch.equal(q, want_q) and torch.equal(s, want_s)
    # and the quantiser against the numpy statement of the scheme
    xq, xs = restate.q_quantize_rows(host(want))
    assert (want_q.cpu().numpy() == xq).all() and maxdiff(host(want_s), xs.reshape(-1)) == 0.0


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("M,N,K", [(300, 3072, 768), (8192, 3072, 768), (128, 3072, 768), (77, 768, 3072), (1000, 200, 64), (2100, 4096, 1024)])
@pytest.mark.parametrize("epi", ["bias_gelu", "bias_residual", "none"])
def test_int8_linear_gathers_row_maxima_for_the_next_quantiser(ctx, dt, M, N, K, epi):
    """ttb_linear_int8_rowmax + ttb_quantize_rows_int8_given_max == ttb_linear_int8 + ttb_quantize_rows_int8, bit for bit
    (every tile shape the dispatcher picks: CTA pairs, single CTAs, narrow tiles, split-K clusters)."""
    r = rng(M + N + K)
    xq = torch.from_numpy(r.integers(-127, 128, (M, K)).astype(np.int8)).cuda()
    xs = torch.from_numpy((r.random(M).astype(np.float32) + 0.5) * 0.02).cuda()
    wq = torch.from_numpy(r.integers(-127, 128, (N, K)).astype(np.int8)).cuda()
    ws = torch.tensor([0.004], dtype=torch.float32, device="cuda")
    bias = dev(r.standard_normal(N).astype(np.float32), dt)
    res = dev(r.standard_normal((M, N)).astype(np.float32), dt)
    e = {"none": 0, "bias_gelu": 2, "bias_residual": 3}[epi]
    want = torch.empty((M, N), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("linear_int8", code(dt), xq, xs, wq, ws, bias, res, N, M, N, K, e, want, N)
    want_q = torch.empty((M, N), dtype=torch.int8, device="cuda")
    want_s = torch.empty(M, dtype=torch.float32, device="cuda")
    ctx.call("quantize_rows_int8", code(dt), want, M, N, want_q, want_s)
    out = torch.empty_like(want)
    amax = torch.full((M,), 1e30, dtype=torch.float32, device="cuda")   # the call overwrites it
    ctx.call("linear_int8_rowmax", code(dt), xq, xs, wq, ws, bias, res, N, M, N, K, e, out, N, amax)
    q = torch.full((M, N), 99, dtype=torch.int8, device="cuda")
    s = torch.full((M,), -1.0, dtype=torch.float32, device="cuda")
    ctx.call("quantize_rows_int8_given_max", code(dt), out, M, N, amax, q, s)
    assert ctx.device_status() == _capi.OK
    assert torch.equal(out, want)
    assert torch.equal(amax, want.float().abs().amax(dim=1))
    assert torch.equal(s, want_s) and torch.equal(q, want_q)
