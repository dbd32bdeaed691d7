"""GPU parity of the primitive C-ABI ops against the numpy restatement of the reference's CPU kernels.

Shapes follow the reference's own unit tests (layers/kernels/*_test.cpp): matmul m in {5,10,15,20} with
n,k in {768,3072}; transposes B in {1,12,20}, L in {10..128}; softmax with 2-D and 3-D masks; layer norm
hidden in {768,2000}; activation hidden in {500,768,8193}; plus empty and ragged inputs.
Tolerances: fp32 1e-4 max-abs (the reference used 1e-3 between its CPU and GPU kernels), fp16 4e-3,
bf16 3e-2 on values of order one.
"""
import numpy as np
import pytest
import torch

from oracle import restate
from tests.helpers import ATOL, TORCH_DT, code, dev, host, maxdiff, rng, rounded
from turbotransformers_b200 import _capi

pytestmark = pytest.mark.gpu
DTS = ["f32", "f16", "bf16"]


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("m", [5, 20])
@pytest.mark.parametrize("n,k", [(768, 3072), (3072, 768)])
@pytest.mark.parametrize("b_trans", [0, 1])
def test_matmul(ctx, dt, m, n, k, b_trans):
    r = rng(1)
    a = rounded(r.random((m, k), np.float32), dt)
    b = rounded(r.random((n, k) if b_trans else (k, n), np.float32), dt)
    want = restate.mat_mul(a, False, b, bool(b_trans))
    A, B, Cc = dev(a, dt), dev(b, dt), dev(np.zeros((m, n), np.float32), dt)
    ctx.call("matmul", code(dt), A, 0, B, b_trans, m, n, k, 1.0, 0.0, Cc)
    # inputs in [0,1): results are about k/4, so the tolerance is relative to that magnitude
    tol = {"f32": 2e-6, "f16": 1e-3, "bf16": 8e-3}[dt] * k
    assert maxdiff(host(Cc), want) < tol


def test_matmul_known_answer(ctx):
    # the literal numbers of layers/kernels/mat_mul_test.cpp:29-47
    A, B = dev(np.array([[1, 2], [3, 4]], np.float32)), dev(np.array([[2, 3], [4, 5]], np.float32))
    Cc = dev(np.zeros((2, 2), np.float32))
    ctx.call("matmul", _capi.F32, A, 0, B, 0, 2, 2, 2, 1.0, 0.0, Cc)
    assert host(Cc).reshape(-1).tolist() == [10, 13, 22, 29]
    ctx.call("matmul", _capi.F32, A, 0, B, 0, 2, 2, 2, 1.0, 1.0, Cc)  # beta accumulates
    assert host(Cc).reshape(-1).tolist() == [20, 26, 44, 58]


@pytest.mark.parametrize("m,n,k", [(70, 100, 37), (1000, 1301, 37), (128, 768, 768)])  # 32 x 32 tiles, 64 x 64 tiles, one request
@pytest.mark.parametrize("a_trans,b_trans", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_matmul_fp32_both_tile_shapes_ragged_sizes(ctx, m, n, k, a_trans, b_trans):
    r = rng(11)
    a = r.standard_normal((k, m) if a_trans else (m, k)).astype(np.float32)
    b = r.standard_normal((n, k) if b_trans else (k, n)).astype(np.float32)
    want = (a.T if a_trans else a).astype(np.float64) @ (b.T if b_trans else b).astype(np.float64)
    A, B, Cc = dev(a), dev(b), dev(np.full((m, n), 7.0, np.float32))
    ctx.call("matmul", _capi.F32, A, a_trans, B, b_trans, m, n, k, 1.0, 0.0, Cc)
    assert np.abs(host(Cc).astype(np.float64) - want).max() < 2e-6 * k * 4
    ctx.call("matmul", _capi.F32, A, a_trans, B, b_trans, m, n, k, 0.5, 2.0, Cc)  # alpha and beta
    assert np.abs(host(Cc).astype(np.float64) - 2.5 * want).max() < 2e-6 * k * 10


@pytest.mark.parametrize("batch,L", [(40, 509), (12, 250)])  # 128 x 128 tiles and 64 x 128 tiles with a ragged last tile
def test_batch_matmul_fp32_ragged_attention_scores_on_the_wide_tiles(ctx, batch, L):
    r = rng(12)
    q = r.standard_normal((batch, L, 64)).astype(np.float32)
    k = r.standard_normal((batch, L, 64)).astype(np.float32)
    want = np.einsum("bld,bmd->blm", q.astype(np.float64), k.astype(np.float64)) * 0.125
    Q, K, S = dev(q), dev(k), dev(np.full((batch, L, L), 3.0, np.float32))
    ctx.call("batch_matmul", _capi.F32, Q, 0, K, 1, batch, L, L, 64, 0.125, 0.0, S)
    assert np.abs(host(S).astype(np.float64) - want).max() < 2e-5


@pytest.mark.parametrize("dt", DTS)
def test_batch_matmul_attention_shapes(ctx, dt):
    r = rng(2)
    B, h, L, d = 2, 3, 37, 64
    q = rounded(r.standard_normal((B, h, L, d)).astype(np.float32), dt)
    k = rounded(r.standard_normal((B, h, L, d)).astype(np.float32), dt)
    want = restate.batch_mat_mul(q, False, k, True, 0.125)
    Q, K, S = dev(q, dt), dev(k, dt), dev(np.zeros((B, h, L, L), np.float32), dt)
    ctx.call("batch_matmul", code(dt), Q, 0, K, 1, B * h, L, L, d, 0.125, 0.0, S)
    assert maxdiff(host(S), want) < ATOL[dt] * 8
    p = rounded(r.random((B, h, L, L)).astype(np.float32), dt)
    want2 = restate.batch_mat_mul(p, False, k, False, 1.0)
    P, O = dev(p, dt), dev(np.zeros((B, h, L, d), np.float32), dt)
    ctx.call("batch_matmul", code(dt), P, 0, K, 0, B * h, L, d, L, 1.0, 0.0, O)
    assert maxdiff(host(O), want2) < ATOL[dt] * 16


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("B,L,heads,d", [(1, 10, 12, 64), (12, 32, 12, 64), (20, 128, 12, 64), (2, 7, 3, 40)])
def test_split_add_bias_transpose_and_back(ctx, dt, B, L, heads, d):
    r = rng(3)
    H = heads * d
    qkv = rounded(r.random((B, L, 3, H), np.float32), dt)
    bias = rounded(r.random((3 * H,), np.float32), dt)
    wq, wk, wv = restate.split_add_bias_transpose_for_score(qkv, bias, heads)
    Q, K, V = (dev(np.zeros((B, heads, L, d), np.float32), dt) for _ in range(3))
    ctx.call("split_add_bias_transpose", code(dt), dev(qkv, dt), dev(bias, dt), B, L, heads, d, Q, K, V)
    for got, want in ((Q, wq), (K, wk), (V, wv)):
        assert maxdiff(host(got), want) < ATOL[dt]
    back = dev(np.zeros((B, L, H), np.float32), dt)
    ctx.call("transpose_for_score", code(dt), Q, B, heads, L, d, back)
    assert maxdiff(host(back), restate.transpose_for_score(host(Q))) == 0.0
    x = rounded(r.random((B, L, heads, d), np.float32), dt)
    b1 = rounded(r.random((H,), np.float32), dt)
    out = dev(np.zeros((B, heads, L, d), np.float32), dt)
    ctx.call("add_bias_transpose_for_score", code(dt), dev(x, dt), dev(b1, dt), B, L, heads, d, out)
    assert maxdiff(host(out), restate.add_bias_transpose_for_score(x, b1)) < ATOL[dt]


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("seq_list", [[4, 7, 2], [9, 7, 13], [1], [37, 5, 128, 64]])
def test_pad_family_matches_reference_semantics(ctx, dt, seq_list):
    # the sequence lists of transpose_test.cpp:138-216 and multi_head_attn_smart_batch_test.py:155-165
    r = rng(4)
    heads, d = 4, 64
    H = heads * d
    B, maxL, T = len(seq_list), max(seq_list), sum(seq_list)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(seq_list)]), dtype=torch.int32).cuda()
    qkv = rounded(r.random((1, T, 3, H), np.float32), dt)
    bias = rounded(r.random((3 * H,), np.float32), dt)
    wq, wk, wv = restate.split_add_bias_transpose_for_score_pad(qkv, bias, heads, seq_list)
    Q, K, V = (dev(np.full((B, heads, maxL, d), 7.0, np.float32), dt) for _ in range(3))
    ctx.call("split_add_bias_transpose_pad", code(dt), dev(qkv, dt), dev(bias, dt), cu, B, maxL, heads, d, Q, K, V)
    for got, want in ((Q, wq), (K, wk), (V, wv)):
        assert maxdiff(host(got), want) < ATOL[dt]  # includes the zero fill of the padding
    packed = dev(np.zeros((1, T, H), np.float32), dt)
    ctx.call("transpose_for_score_pad", code(dt), Q, cu, B, maxL, heads, d, packed)
    assert maxdiff(host(packed), restate.transpose_for_score_pad(host(Q), seq_list)) == 0.0
    x = rounded(r.random((1, T, heads, d), np.float32), dt)
    b1 = rounded(r.random((H,), np.float32), dt)
    out = dev(np.full((B, heads, maxL, d), 7.0, np.float32), dt)
    ctx.call("add_bias_transpose_for_score_pad", code(dt), dev(x, dt), dev(b1, dt), cu, B, maxL, heads, d, out)
    assert maxdiff(host(out), restate.add_bias_transpose_for_score_pad(x, b1, seq_list)) < ATOL[dt]


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("B,heads,Lq,Lk,mask_kind", [(1, 12, 10, 10, "2d"), (20, 12, 40, 100, "2d"), (2, 4, 500, 70, "3d"),
                                                      (2, 2, 33, 1500, "none"), (3, 2, 16, 16, "3d")])
def test_mask_softmax(ctx, dt, B, heads, Lq, Lk, mask_kind):
    r = rng(5)
    s = rounded(r.standard_normal((B, heads, Lq, Lk)).astype(np.float32) * 3, dt)
    mask = None
    if mask_kind == "2d":
        mask = np.where(r.random((B, 1, 1, Lk)) < 0.2, -10000.0, 0.0).astype(np.float32)
        mask[..., 0] = 0
    elif mask_kind == "3d":
        mask = np.where(r.random((B, Lq, Lk)) < 0.3, -1e9, 0.0).astype(np.float32)
        mask[..., 0] = 0
    want = restate.apply_mask_and_softmax(s, mask, 0.5)
    S = dev(s, dt)
    M = dev(mask) if mask is not None else None
    ctx.call("mask_softmax", code(dt), S, M, B, heads, Lq, Lk, 0.5, 1 if mask_kind == "2d" else 0)
    assert maxdiff(host(S), want) < {"f32": 1e-5, "f16": 1e-3, "bf16": 8e-3}[dt]
    assert abs(host(S).sum(-1) - 1).max() < {"f32": 1e-5, "f16": 2e-2, "bf16": 1e-1}[dt]


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("M,N", [(1, 768), (20 * 128, 768), (37, 2000), (5, 1024), (3, 4096), (9, 100), (0, 768)])
def test_layernorm_and_add_bias_layernorm(ctx, dt, M, N):
    r = rng(6)
    out = rounded(r.standard_normal((M, N)).astype(np.float32), dt)
    inp = rounded(r.standard_normal((M, N)).astype(np.float32), dt)
    bias, gamma, beta = (rounded(r.standard_normal(N).astype(np.float32), dt) for _ in range(3))
    want = restate.add_bias_layer_norm(inp, bias, gamma, beta, out, 1e-12)
    O = dev(out, dt)
    ctx.call("add_bias_layernorm", code(dt), O, dev(inp, dt), dev(bias, dt), dev(gamma, dt), dev(beta, dt), M, N, 1e-12)
    assert maxdiff(host(O), want) < ATOL[dt] * 4
    want2 = restate.layer_norm(out, gamma, beta, 1e-5)
    X, Y = dev(out, dt), dev(np.zeros((M, N), np.float32), dt)
    ctx.call("layernorm", code(dt), X, Y, dev(gamma, dt), dev(beta, dt), M, N, 1e-5)
    assert maxdiff(host(Y), want2) < ATOL[dt] * 4
    ctx.call("layernorm", code(dt), X, X, dev(gamma, dt), dev(beta, dt), M, N, 1e-5)  # in place
    assert maxdiff(host(X), want2) < ATOL[dt] * 4


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("M,N", [(1184, 768), (1185, 768), (4735, 768), (4737, 768), (18424, 768), (9999, 1024), (20001, 256), (6000, 520)])
def test_layernorm_16bit_every_kernel_by_row_count(ctx, dt, M, N):
    """The 16-bit LayerNorm picks its kernel by row count (one row per warp / register streaming / bulk-copy staged);
    sizes on both sides of each switch, ragged last chunks, in place and out of place, all against the restatement."""
    r = rng(M + N)
    x = rounded(r.standard_normal((M, N)).astype(np.float32) * 1.5 + 0.25, dt)
    gamma, beta = (rounded(r.standard_normal(N).astype(np.float32), dt) for _ in range(2))
    want = restate.layer_norm(x, gamma, beta, 1e-12)
    X = dev(x, dt)
    Y = torch.full((M + 1, N), float("nan"), dtype=TORCH_DT[dt], device="cuda")   # one guard row behind the output
    ctx.call("layernorm", code(dt), X, Y, dev(gamma, dt), dev(beta, dt), M, N, 1e-12)
    assert ctx.device_status() == _capi.OK
    assert torch.isnan(Y[M]).all()
    assert maxdiff(host(Y[:M]), want) < ATOL[dt] * 4
    ctx.call("layernorm", code(dt), X, X, dev(gamma, dt), dev(beta, dt), M, N, 1e-12)
    assert torch.equal(X, Y[:M])


def test_layernorm_honours_eps(ctx):
    # a constant row has zero variance: the result is beta only if eps enters the rsqrt
    x = dev(np.full((2, 768), 3.0, np.float32))
    g, b = dev(np.ones(768, np.float32)), dev(np.full(768, 0.25, np.float32))
    ctx.call("layernorm", _capi.F32, x, x, g, b, 2, 768, 1e-12)
    assert np.isfinite(host(x)).all() and maxdiff(host(x), 0.25) < 1e-3


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("M,N", [(10, 500), (128, 768), (3, 8193), (64, 3072)])
@pytest.mark.parametrize("act", ["gelu", "tanh", "relu"])
def test_add_bias_act(ctx, dt, M, N, act):
    r = rng(7)
    x = rounded(r.standard_normal((M, N)).astype(np.float32) * 2, dt)
    bias = rounded(r.standard_normal(N).astype(np.float32), dt)
    want = restate.add_bias_act(x, bias, act)
    X = dev(x, dt)
    ctx.call("add_bias_act", code(dt), X, dev(bias, dt), M, N, {"gelu": 0, "tanh": 1, "relu": 2}[act])
    assert maxdiff(host(X), want) < ATOL[dt] * 4


@pytest.mark.parametrize("dt", DTS)
def test_bias_adds(ctx, dt):
    r = rng(8)
    M, N = 33, 768
    a, b = (rounded(r.standard_normal((M, N)).astype(np.float32), dt) for _ in range(2))
    bias = rounded(r.standard_normal(N).astype(np.float32), dt)
    A = dev(a, dt)
    ctx.call("add_bias", code(dt), A, dev(bias, dt), M, N)
    assert maxdiff(host(A), restate.add_bias(a, bias)) < ATOL[dt] * 2
    O = dev(np.zeros((M, N), np.float32), dt)
    ctx.call("add_input_bias", code(dt), dev(a, dt), dev(b, dt), dev(bias, dt), M, N, O)
    assert maxdiff(host(O), restate.add_input_bias(a, b, bias)) < ATOL[dt] * 4


@pytest.mark.parametrize("dt", DTS)
def test_lookup_embedding_set_and_add(ctx, dt):
    r = rng(9)
    vocab, hidden, n = 300, 768, 50
    table = rounded(r.standard_normal((vocab, hidden)).astype(np.float32), dt)
    ids = r.integers(0, vocab, n).astype(np.int64)
    out = dev(np.zeros((n, hidden), np.float32), dt)
    ctx.call("lookup_embedding", code(dt), out, dev(table, dt), dev(ids), n, hidden, vocab, 0)
    assert maxdiff(host(out), restate.lookup_embedding(table, ids)) == 0.0
    ctx.call("lookup_embedding", code(dt), out, dev(table, dt), dev(ids), n, hidden, vocab, 1)
    assert maxdiff(host(out), rounded(restate.lookup_embedding(table, ids) * 2, dt)) < ATOL[dt]
    assert ctx.device_status() == _capi.OK


def test_lookup_embedding_bad_id_is_flagged_not_trapped(ctx):
    table = dev(np.arange(40, dtype=np.float32).reshape(10, 4))
    ids = dev(np.array([3, 99, -1], np.int64))
    out = dev(np.zeros((3, 4), np.float32))
    ctx.call("lookup_embedding", _capi.F32, out, table, ids, 3, 4, 10, 0)
    assert ctx.device_status() == _capi.ERR_BAD_INDEX
    assert host(out)[0].tolist() == [12, 13, 14, 15] and host(out)[1].tolist() == [36, 37, 38, 39]
    assert ctx.device_status() == _capi.OK  # the word is cleared by the read; the context stays usable


@pytest.mark.parametrize("dt", DTS)
@pytest.mark.parametrize("pool", ["First", "Last", "Mean", "Max"])
def test_seq_pool(ctx, dt, pool):
    r = rng(10)
    B, L, H = 3, 17, 768
    x = rounded(r.standard_normal((B, L, H)).astype(np.float32), dt)
    out = dev(np.zeros((B, H), np.float32), dt)
    ctx.call("seq_pool", code(dt), dev(x, dt), B, L, H, ["First", "Last", "Mean", "Max"].index(pool), out)
    assert maxdiff(host(out), restate.seq_pool(x, pool)) < ATOL[dt]
    lens = [5, 9, 3]
    cu = torch.tensor([0, 5, 14, 17], dtype=torch.int32).cuda()
    packed = x.reshape(-1, H)[:17]
    out2 = dev(np.zeros((3, H), np.float32), dt)
    ctx.call("seq_pool_varlen", code(dt), dev(packed, dt), cu, 3, H, ["First", "Last", "Mean", "Max"].index(pool), out2)
    want = np.stack([restate.seq_pool(packed[None, s:s + n], pool)[0] for s, n in zip([0, 5, 14], lens)])
    assert maxdiff(host(out2), want) < ATOL[dt]


def test_prepare_bert_masks(ctx):
    B, L = 3, 11
    r = rng(11)
    mask_in = (r.random((B, L)) > 0.3).astype(np.int64)
    am, tt, pos = (torch.full((B, L), -5, dtype=torch.int64).cuda() for _ in range(3))
    ext = torch.zeros(B, L).cuda()
    ctx.call("prepare_bert_masks", B, L, dev(mask_in), am, tt, pos, ext)
    wam, wtt, wpos, wext = restate.prepare_bert_masks(np.zeros((B, L), np.int64), mask_in)
    assert (am.cpu().numpy() == wam).all() and (tt.cpu().numpy() == wtt).all() and (pos.cpu().numpy() == wpos).all()
    assert maxdiff(host(ext), wext.reshape(B, L)) == 0.0
    ctx.call("prepare_bert_masks", B, L, None, am, None, None, ext)  # defaults: all ones -> zeros
    assert (am.cpu().numpy() == 1).all() and host(ext).max() == 0.0


@pytest.mark.parametrize("dt", DTS)
def test_embedding_ln_fixed_and_varlen(ctx, dt):
    r = rng(12)
    vocab, npos, ntype, H = 500, 64, 2, 768
    w = {"word": rounded(r.standard_normal((vocab, H)).astype(np.float32) * 0.02, dt),
         "position": rounded(r.standard_normal((npos, H)).astype(np.float32) * 0.02, dt),
         "token_type": rounded(r.standard_normal((ntype, H)).astype(np.float32) * 0.02, dt),
         "ln_gamma": rounded(1 + 0.1 * r.standard_normal(H).astype(np.float32), dt),
         "ln_beta": rounded(0.1 * r.standard_normal(H).astype(np.float32), dt)}
    D = {k: dev(v, dt) for k, v in w.items()}
    B, L = 3, 20
    ids = r.integers(0, vocab, (B, L)).astype(np.int64)
    _, tt, pos, _ = restate.prepare_bert_masks(ids)
    want = restate.bert_embedding(ids, pos, tt, w)
    out = dev(np.zeros((B, L, H), np.float32), dt)
    ctx.call("embedding_ln", code(dt), dev(ids), None, None, None, B, L, B * L, D["word"], D["position"], D["token_type"],
             D["ln_gamma"], D["ln_beta"], H, vocab, npos, ntype, 1e-12, out)
    assert maxdiff(host(out), want) < ATOL[dt] * 4
    lens = [7, 20, 1, 12]
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32).cuda()
    flat = r.integers(0, vocab, sum(lens)).astype(np.int64)
    parts, s = [], 0
    for n in lens:
        i = flat[s:s + n][None]
        _, tt, pos, _ = restate.prepare_bert_masks(i)
        parts.append(restate.bert_embedding(i, pos, tt, w)[0])
        s += n
    out2 = dev(np.zeros((sum(lens), H), np.float32), dt)
    ctx.call("embedding_ln", code(dt), dev(flat), None, None, cu, len(lens), 0, sum(lens), D["word"], D["position"],
             D["token_type"], D["ln_gamma"], D["ln_beta"], H, vocab, npos, ntype, 1e-12, out2)
    assert maxdiff(host(out2), np.concatenate(parts)) < ATOL[dt] * 4
    assert ctx.device_status() == _capi.OK


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("H", [256, 512, 1024, 264, 100])
def test_embedding_ln_16bit_widths_and_explicit_ids(ctx, dt, H):
    """Every width the 16-byte-vector kernel is instantiated for (and two it is not: 264 > 256 takes the next size up, 100
    is not a multiple of 8), with caller-supplied position and token-type ids and one id out of range (clamped, flagged)."""
    r = rng(H)
    vocab, npos, ntype = 300, 40, 3
    w = {"word": rounded(r.standard_normal((vocab, H)).astype(np.float32) * 0.05, dt),
         "position": rounded(r.standard_normal((npos, H)).astype(np.float32) * 0.05, dt),
         "token_type": rounded(r.standard_normal((ntype, H)).astype(np.float32) * 0.05, dt),
         "ln_gamma": rounded(1 + 0.1 * r.standard_normal(H).astype(np.float32), dt),
         "ln_beta": rounded(0.1 * r.standard_normal(H).astype(np.float32), dt)}
    D = {k: dev(v, dt) for k, v in w.items()}
    B, L = 5, 33
    ids = r.integers(0, vocab, (B, L)).astype(np.int64)
    pos = r.integers(0, npos, (B, L)).astype(np.int64)
    tt = r.integers(0, ntype, (B, L)).astype(np.int64)
    want = restate.bert_embedding(ids, pos, tt, w)
    out = torch.full((B * L + 1, H), float("nan"), dtype=TORCH_DT[dt], device="cuda")
    ctx.call("embedding_ln", code(dt), dev(ids), dev(pos), dev(tt), None, B, L, B * L, D["word"], D["position"], D["token_type"],
             D["ln_gamma"], D["ln_beta"], H, vocab, npos, ntype, 1e-12, out)
    assert ctx.device_status() == _capi.OK
    assert torch.isnan(out[B * L]).all()
    assert maxdiff(host(out[:B * L]).reshape(B, L, H), want) < ATOL[dt] * 4
    bad = ids.copy()
    bad[2, 7] = vocab + 5
    ctx.call("embedding_ln", code(dt), dev(bad), dev(pos), dev(tt), None, B, L, B * L, D["word"], D["position"], D["token_type"],
             D["ln_gamma"], D["ln_beta"], H, vocab, npos, ntype, 1e-12, out)
    assert ctx.device_status() == _capi.ERR_BAD_INDEX      # reading the status also clears it
    clamped = ids.copy()
    clamped[2, 7] = vocab - 1
    assert maxdiff(host(out[:B * L]).reshape(B, L, H), restate.bert_embedding(clamped, pos, tt, w)) < ATOL[dt] * 4
    assert ctx.device_status() == _capi.OK


def test_invalid_arguments_return_status_without_launching(ctx):
    lib = _capi.lib()
    before = ctx.launches()
    assert lib.ttb_layernorm(ctx.h, _capi.F32, None, None, None, None, 4, 768, 1e-12) == _capi.ERR_INVALID
    assert lib.ttb_layernorm(ctx.h, 9, None, None, None, None, 0, 768, 1e-12) in (_capi.OK, _capi.ERR_UNSUPPORTED)
    assert lib.ttb_add_bias_act(ctx.h, _capi.F32, None, None, 4, 8, 7) == _capi.ERR_INVALID
    assert lib.ttb_matmul(ctx.h, _capi.F32, None, 0, None, 0, -1, 2, 2, 1.0, 0.0, None) == _capi.ERR_INVALID
    assert b"" != lib.ttb_last_error(ctx.h)
    assert ctx.launches() == before


def test_allocator_pool_contract(ctx):
    import ctypes as C
    lib = _capi.lib()
    ptr, in_use, hw, n = C.c_void_p(), C.c_size_t(), C.c_size_t(), C.c_uint64()
    lib.ttb_pool_stats(ctx.h, C.byref(in_use), C.byref(hw), C.byref(n))
    base = in_use.value
    assert lib.ttb_alloc(ctx.h, 1 << 20, b"test/buf", C.byref(ptr)) == _capi.OK and ptr.value
    lib.ttb_pool_stats(ctx.h, C.byref(in_use), C.byref(hw), C.byref(n))
    assert in_use.value == base + (1 << 20) and hw.value >= in_use.value
    assert lib.ttb_free(ctx.h, ptr, b"test/buf") == _capi.OK
    assert lib.ttb_free(ctx.h, ptr, b"test/buf") == _capi.ERR_INVALID  # double free is reported, not fatal
    # exhaustion through a tiny cap: an error code, not an abort
    assert lib.ttb_pool_set_limit(ctx.h, base + 4096) == _capi.OK
    assert lib.ttb_alloc(ctx.h, 1 << 20, b"test/too_big", C.byref(ptr)) == _capi.ERR_OOM and not ptr.value
    assert lib.ttb_pool_set_limit(ctx.h, 0) == _capi.OK
    arena = C.c_size_t()
    assert lib.ttb_plan_activations(ctx.h, 1, 128, 12, 768, 3072, 12, _capi.F16, C.byref(arena)) == _capi.OK
    assert arena.value >= 128 * (7 * 768 + 3072) * 2


def test_bounded_device_wait_gives_up_and_is_reported(ctx):
    """The mbarrier waits of the tensor-core kernels are bounded; here one is made to run out (a barrier nothing arrives
    at, a limit of about a millisecond). It must return by itself with the abort flag set, and the status word must carry
    TTB_ERR_DEVICE_WAIT until it is read."""
    assert ctx.device_status() == _capi.OK
    observed = torch.full((3,), -1, dtype=torch.int32, device="cuda")
    limit = 1_000_000
    ctx.call("selftest_bounded_wait", limit, observed)
    status = ctx.device_status()           # synchronises: the kernel has returned
    completed, aborted, kcycles = observed.cpu().tolist()
    assert completed == 0 and aborted == 1
    assert limit // 1024 <= kcycles < 50 * limit // 1024   # it waited out its limit and not much more
    assert status == _capi.ERR_DEVICE_WAIT
    assert b"bounded device-side wait" in _capi.lib().ttb_last_error(ctx.h)
    assert ctx.device_status() == _capi.OK  # reading the status cleared it; the context stays usable
    x = torch.ones(4, 8, device="cuda", dtype=torch.float16)
    ctx.call("add_bias", _capi.F16, x, torch.ones(8, device="cuda", dtype=torch.float16), 4, 8)
    assert float(x.sum().item()) == 64.0
    with pytest.raises(_capi.TTBError):
        ctx.call("selftest_bounded_wait", 10**10, observed)  # limits beyond a twentieth of a second are refused
