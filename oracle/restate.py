"""TEST INFRASTRUCTURE ONLY -- a numpy fp32 restatement of the reference's CPU algorithm for the
transformer-layer forward path.  Nothing in the product package may import this file; it exists so the
CUDA path can be checked on arbitrary shapes, also where the compiled reference (oracle/_ref) is absent.

Parity status: PINNED.  tests/test_oracle_pinning.py checks every function here against (a) the golden
vectors under tests/golden/ that were produced by the compiled, unmodified reference CPU code
(oracle/_ref, see tests/golden/make_golden.py) and (b) the literal known-answer numbers in the
reference's own unit tests (mat_mul_test.cpp:29-77, transpose_test.cpp pad-vs-unpadded semantics).
The `q_*` functions restate the benchmark's own int8 scheme (all six Linears, per-row activation scales), which the
reference does not implement: that part is "parity unpinned" against reference code and is pinned bit-exactly only at
kernel level.  The `qref_*` functions restate the reference's recipe (torch dynamic quantisation of the two feed-forward
Linears); they are pinned against the installed torch's quantised Linear and against the golden vector that recipe
produced through the compiled reference's epilogues.

All citations are paths inside the reference project (turbo_transformers/...).
"""
import math

import numpy as np

F32 = np.float32


# --------------------------------------------------------------------------------------------------
# A1 / A2: GEMM wrappers
# --------------------------------------------------------------------------------------------------
def mat_mul(a, a_trans, b, b_trans, alpha=1.0, out=None, beta=0.0):
    """layers/kernels/mat_mul.cpp:30-118 -- A is flattened to [numel/K, K]; out = alpha*op(A)*op(B) + beta*out."""
    a2 = a.reshape(-1, a.shape[-1]).astype(F32)
    a2 = a2.T if a_trans else a2
    b2 = b.T if b_trans else b
    r = F32(alpha) * (a2 @ b2.astype(F32))
    if out is not None and beta != 0.0:
        r = r + F32(beta) * out.reshape(r.shape)
    return r.astype(F32)


def batch_mat_mul(a, a_trans, b, b_trans, alpha=1.0):
    """layers/kernels/mat_mul.cpp:119-213 -- strided batched GEMM over the leading dims."""
    a2 = np.swapaxes(a, -1, -2) if a_trans else a
    b2 = np.swapaxes(b, -1, -2) if b_trans else b
    return (F32(alpha) * np.matmul(a2.astype(F32), b2.astype(F32))).astype(F32)


# --------------------------------------------------------------------------------------------------
# A3 / A5 / S1: transposes
# --------------------------------------------------------------------------------------------------
def split_add_bias_transpose_for_score(qkv, bias, num_heads):
    """layers/kernels/transpose.cpp:310-406 -- [B,L,3,H] + bias[3H] -> q,k,v each [B,h,L,d]."""
    B, L = qkv.shape[0], qkv.shape[1]
    H = qkv.shape[-1]
    d = H // num_heads
    x = qkv.reshape(B, L, 3, num_heads, d) + bias.reshape(1, 1, 3, num_heads, d)
    x = np.transpose(x, (2, 0, 3, 1, 4)).astype(F32)
    return np.ascontiguousarray(x[0]), np.ascontiguousarray(x[1]), np.ascontiguousarray(x[2])


def transpose_for_score(x):
    """layers/kernels/transpose.cpp:158-191 -- [B,h,L,d] -> [B,L,h*d]."""
    B, h, L, d = x.shape
    return np.ascontiguousarray(np.transpose(x, (0, 2, 1, 3))).reshape(B, L, h * d)


def add_bias_transpose_for_score(x, bias):
    """layers/kernels/transpose.cpp:193-240 -- [B,L,h,d] + bias[h*d] -> [B,h,L,d]."""
    B, L, h, d = x.shape
    return np.ascontiguousarray(np.transpose(x + bias.reshape(1, 1, h, d), (0, 2, 1, 3))).astype(F32)


def split_add_bias_transpose_for_score_pad(qkv, bias, num_heads, seq_list):
    """layers/kernels/transpose.cpp:457-580 -- packed [1,sumL,3,H] -> zero-padded q,k,v [B,h,maxL,d]."""
    H = qkv.shape[-1]
    d = H // num_heads
    B, maxL = len(seq_list), max(seq_list)
    out = np.zeros((3, B, num_heads, maxL, d), F32)
    x = qkv.reshape(-1, 3, num_heads, d) + bias.reshape(1, 3, num_heads, d)
    acc = 0
    for b, n in enumerate(seq_list):
        out[:, b, :, :n, :] = np.transpose(x[acc:acc + n], (1, 2, 0, 3))
        acc += n
    return out[0], out[1], out[2]


def transpose_for_score_pad(x, seq_list):
    """layers/kernels/transpose.cpp:582-623 (+ TransposeForScorePadImpl :66-102) -- padded [B,h,maxL,d] -> packed [1,sumL,h*d]."""
    B, h, maxL, d = x.shape
    rows = [np.transpose(x[b, :, :n, :], (1, 0, 2)).reshape(n, h * d) for b, n in enumerate(seq_list)]
    return np.concatenate(rows, 0)[None].astype(F32)


def add_bias_transpose_for_score_pad(x, bias, seq_list):
    """layers/kernels/transpose.cpp:409-440 (+ Impl :128-156) -- packed [1,sumL,h,d] + bias -> padded [B,h,maxL,d]."""
    _, _, h, d = x.shape
    B, maxL = len(seq_list), max(seq_list)
    out = np.zeros((B, h, maxL, d), F32)
    acc = 0
    xb = x[0] + bias.reshape(1, h, d)
    for b, n in enumerate(seq_list):
        out[b, :, :n, :] = np.transpose(xb[acc:acc + n], (1, 0, 2))
        acc += n
    return out


# --------------------------------------------------------------------------------------------------
# A4: mask + softmax
# --------------------------------------------------------------------------------------------------
def apply_mask_and_softmax(scores, mask, scale=1.0):
    """layers/kernels/softmax.cpp:28-125 -- in-place softmax(scores*scale + mask) over the last dim.

    mask is None, 2-D-like ([B,to], [B,1,to], [B,1,1,to]: one row per batch) or 3-D-like
    ([B,from,to] / [B,1,from,to]: one row per query), chosen exactly as softmax.cpp:93-102 does.
    """
    B, h, Lq, Lk = scores.shape
    s = scores.astype(F32) * F32(scale)
    if mask is not None:
        m = np.asarray(mask, F32)
        two_d = m.ndim == 2 or (m.ndim == 3 and m.shape[1] == 1) or (m.ndim == 4 and m.shape[2] == 1)
        if two_d:
            s = s + m.reshape(B, 1, 1, Lk)
        else:
            s = s + m.reshape(B, 1, Lq, Lk)
    s = s - s.max(-1, keepdims=True)
    e = np.exp(s, dtype=F32)
    return (e * (F32(1.0) / e.sum(-1, keepdims=True, dtype=F32))).astype(F32)


# --------------------------------------------------------------------------------------------------
# A6 / A7: layer norm
# --------------------------------------------------------------------------------------------------
def layer_norm(x, gamma, beta, eps=1e-12):
    """layers/kernels/layer_norm.cpp:32-91 -- var = E[x^2] - mean^2, out = beta + gamma*rsqrt(var+eps)*(x-mean)."""
    x = x.astype(F32)
    n = x.shape[-1]
    mean = x.sum(-1, keepdims=True, dtype=F32) / F32(n)
    var = (x * x).sum(-1, keepdims=True, dtype=F32) / F32(n) - mean * mean
    r = F32(1.0) / np.sqrt(var + F32(eps), dtype=F32)
    return (beta + gamma * r * (x - mean)).astype(F32)


def add_bias_layer_norm(inp, bias, gamma, beta, out, eps=1e-12):
    """layers/kernels/layer_norm.cpp:98-180 -- out = LN(out + input + bias)*gamma + beta."""
    return layer_norm(out.astype(F32) + inp.astype(F32) + bias.astype(F32), gamma, beta, eps)


# --------------------------------------------------------------------------------------------------
# A8: bias + activation
# --------------------------------------------------------------------------------------------------
def gelu_tanh(x):
    """layers/kernels/activation.cpp:32-55 -- 0.5*x*(1+tanh(0.7978845608*(x+0.044715*x^3)))."""
    x = x.astype(F32)
    return (x * F32(0.5) * (F32(1.0) + np.tanh(F32(0.7978845608028654) * (x + F32(0.044715) * x * x * x)))).astype(F32)


def add_bias_act(x, bias, act):
    """layers/kernels/activation.cpp:90-119 -- in-place act(x + bias); act in {'gelu','tanh','relu'}."""
    y = x.astype(F32) + bias.astype(F32)
    if act == "gelu":
        return gelu_tanh(y)
    if act == "tanh":
        return np.tanh(y).astype(F32)
    if act == "relu":
        return np.maximum(y, F32(0))
    raise ValueError(act)


# --------------------------------------------------------------------------------------------------
# A9-A12: embedding, bias adds, pooling, mask preparation
# --------------------------------------------------------------------------------------------------
def lookup_embedding(table, ids, out=None):
    """layers/kernels/embedding.cpp:28-85 -- out[i,:] (=|+=) table[ids[i],:]."""
    g = table[np.asarray(ids).reshape(-1)]
    g = g.reshape(tuple(np.asarray(ids).shape) + (table.shape[1],)).astype(F32)
    return g if out is None else (out + g).astype(F32)


def add_bias(x, bias):
    """layers/kernels/utils.cpp:103-131 -- x += bias."""
    return (x + bias).astype(F32)


def add_input_bias(in1, in2, bias):
    """layers/kernels/utils.cpp:134-169 -- out = in1 + in2 + bias."""
    return (in1 + in2 + bias).astype(F32)


def seq_pool(x, pool_type):
    """layers/kernels/seq_pool.cpp:124-155 -- First/Last/Mean/Max over the sequence axis of [B,L,H]."""
    if pool_type == "First":
        return np.ascontiguousarray(x[:, 0, :])
    if pool_type == "Last":
        return np.ascontiguousarray(x[:, -1, :])
    if pool_type == "Mean":
        return (x.sum(1, dtype=F32) / F32(x.shape[1])).astype(F32)
    if pool_type == "Max":
        return x.max(1)
    raise ValueError(pool_type)


def prepare_bert_masks(ids, att_mask=None, token_type=None, position_ids=None):
    """layers/prepare_bert_masks.cpp:24-66 + kernels/common.cpp:37-90.

    Returns (att_mask int64 [B,L], token_type int64, position_ids int64, extended fp32 [B,1,1,L] = -10000*(1-mask)).
    """
    B, L = ids.shape
    if position_ids is None:
        position_ids = np.tile(np.arange(L, dtype=np.int64), (B, 1))
    if token_type is None:
        token_type = np.zeros((B, L), np.int64)
    if att_mask is None:
        att_mask = np.ones((B, L), np.int64)
    ext = (F32(-10000.0) * (F32(1.0) - att_mask.astype(F32))).reshape(B, 1, 1, L)
    return att_mask, token_type, position_ids, ext


# --------------------------------------------------------------------------------------------------
# L1-L5: layers
# --------------------------------------------------------------------------------------------------
def multi_headed_attention(x, mask, w, num_heads, pre_layernorm=False, post_layernorm=False,
                           post_add_input=False, pre_ln_eps=1e-6):
    """Self-attention branch of layers/multi_headed_attention.cpp:168-232,260-380.

    w: dict with qkv_weight [H,3H], qkv_bias [3H], dense_weight [H,H], dense_bias [H], ln_gamma, ln_beta.
    Returns (output [B,L,H], att_score [B,h,L,L]).  The reference hard-codes the pre-LN epsilon to 1e-6
    (multi_headed_attention.cpp:194-195); `pre_ln_eps` exposes it because GPT-2 needs 1e-5.
    """
    B, L, H = x.shape
    d = H // num_heads
    q_in = layer_norm(x, w["ln_gamma"], w["ln_beta"], pre_ln_eps) if pre_layernorm else x
    qkv = mat_mul(q_in, False, w["qkv_weight"], False).reshape(B, L, 3, H)
    q, k, v = split_add_bias_transpose_for_score(qkv, w["qkv_bias"], num_heads)
    score = batch_mat_mul(q, False, k, True, 1.0 / math.sqrt(float(d)))
    prob = apply_mask_and_softmax(score, mask, 1.0)
    ctx = transpose_for_score(batch_mat_mul(prob, False, v, False))
    out = mat_mul(ctx, False, w["dense_weight"], False).reshape(B, L, H)
    if not post_add_input:
        if not post_layernorm:
            out = add_bias(out, w["dense_bias"])
        else:
            out = add_bias_layer_norm(x, w["dense_bias"], w["ln_gamma"], w["ln_beta"], out, 1e-12)
    else:
        out = add_input_bias(out, x, w["dense_bias"])
    return out, prob


def context_attention(query, key, value, mask, w, num_heads, memory=None, pre_layernorm=False, post_layernorm=False,
                      post_add_input=False, pre_ln_eps=1e-6):
    """Context (encoder-decoder) branch of layers/multi_headed_attention.cpp:45-167,308-380.

    w: q_weight / k_weight / v_weight [H,H] ([in,out]), q_bias / k_bias / v_bias [H], dense_weight, dense_bias, ln_gamma,
    ln_beta. `memory` = (keys, values) [B,h,Lk,d] as a previous call returned them (layer_cache["memory_keys"/"memory_values"]):
    given, key / value are not projected again. Returns (output [B,Lq,H], att_score [B,h,Lq,Lk], (keys, values)).
    """
    B, Lq, H = query.shape
    d = H // num_heads
    q_in = layer_norm(query, w["ln_gamma"], w["ln_beta"], pre_ln_eps) if pre_layernorm else query
    q = add_bias_transpose_for_score(mat_mul(q_in, False, w["q_weight"], False).reshape(B, Lq, num_heads, d), w["q_bias"])
    if memory is not None:
        k, v = memory
    else:
        Lk = key.shape[1]
        k = add_bias_transpose_for_score(mat_mul(key, False, w["k_weight"], False).reshape(B, Lk, num_heads, d), w["k_bias"])
        v = add_bias_transpose_for_score(mat_mul(value, False, w["v_weight"], False).reshape(B, Lk, num_heads, d), w["v_bias"])
    score = batch_mat_mul(q, False, k, True, 1.0 / math.sqrt(float(d)))
    prob = apply_mask_and_softmax(score, mask, 1.0)
    ctx = transpose_for_score(batch_mat_mul(prob, False, v, False))
    out = mat_mul(ctx, False, w["dense_weight"], False).reshape(B, Lq, H)
    if not post_add_input:
        if not post_layernorm:
            out = add_bias(out, w["dense_bias"])
        else:
            out = add_bias_layer_norm(query, w["dense_bias"], w["ln_gamma"], w["ln_beta"], out, 1e-12)
    else:
        out = add_input_bias(out, query, w["dense_bias"])
    return out, prob, (k, v)


def positionwise_ffn(x, w, eps=1e-12):
    """layers/positionwise_ffn.cpp:31-75 -- LayerNorm(eps 1e-12), MatMul, AddBiasAct<Relu>, MatMul, AddInputBias (residual).
    w: w1_weight [H,F], w1_bias, w2_weight [F,H], w2_bias, ln_gamma, ln_beta ([in,out] matrices)."""
    hdn = layer_norm(x, w["ln_gamma"], w["ln_beta"], eps)
    inter = add_bias_act(mat_mul(hdn, False, w["w1_weight"], False), w["w1_bias"], "relu")
    out = mat_mul(inter, False, w["w2_weight"], False).reshape(x.shape)
    return add_input_bias(out, x, w["w2_bias"])


def transformer_decoder_layer(x, memory_bank, src_mask, dec_mask, lw, num_heads, memory=None):
    """python/turbo_transformers/layers/modeling_decoder.py:58-140 -- pre-LN self attention + residual, pre-LN context attention
    + residual, feed-forward. lw: {"self": multi_headed_attention weights, "context": context_attention weights, "ffn": ...};
    masks are additive (already multiplied by -1e18). Returns (output, context attention of head 0, (memory keys, values))."""
    query, _ = multi_headed_attention(x, dec_mask, lw["self"], num_heads, pre_layernorm=True, post_add_input=True)
    mid, attn, mem = context_attention(query, memory_bank, memory_bank, src_mask, lw["context"], num_heads, memory,
                                       pre_layernorm=True, post_add_input=True)
    return positionwise_ffn(mid, lw["ffn"]), attn[:, 0], mem


def multi_headed_attention_smart_batch(x_packed, seq_list, w, num_heads, mask=None, post_layernorm=True):
    """Self-attention branch of layers/multi_headed_attention_smart_batch.cpp:180-421 on packed [1,sumL,H]."""
    H = x_packed.shape[-1]
    d = H // num_heads
    B, maxL = len(seq_list), max(seq_list)
    if mask is None:  # python/turbo_transformers/layers/modeling_smart_pad.py:82-98
        mask = np.zeros((B, 1, maxL), F32)
        for b, n in enumerate(seq_list):
            mask[b, 0, n:] = -1e9
    qkv = mat_mul(x_packed, False, w["qkv_weight"], False).reshape(1, -1, 3, H)
    q, k, v = split_add_bias_transpose_for_score_pad(qkv, w["qkv_bias"], num_heads, seq_list)
    score = batch_mat_mul(q, False, k, True, 1.0 / math.sqrt(float(d)))
    prob = apply_mask_and_softmax(score, mask, 1.0)
    ctx = transpose_for_score_pad(batch_mat_mul(prob, False, v, False), seq_list)
    out = mat_mul(ctx, False, w["dense_weight"], False).reshape(x_packed.shape)
    if post_layernorm:
        out = add_bias_layer_norm(x_packed, w["dense_bias"], w["ln_gamma"], w["ln_beta"], out, 1e-12)
    else:
        out = add_bias(out, w["dense_bias"])
    return out, prob


def bert_intermediate(x, weight, bias):
    """layers/bert_intermediate.cpp:32-50 -- MatMul [M,H]x[H,F] then AddBiasAct<Gelu>."""
    return add_bias_act(mat_mul(x, False, weight, False), bias, "gelu").reshape(x.shape[:-1] + (weight.shape[1],))


def bert_output(hidden, residual, weight, bias, gamma, beta):
    """layers/bert_output.cpp:29-55 -- MatMul [M,F]x[F,H] then AddBiasLayerNorm(residual, eps=1e-12)."""
    out = mat_mul(hidden, False, weight, False).reshape(residual.shape)
    return add_bias_layer_norm(residual, bias, gamma, beta, out, 1e-12)


def bert_embedding(ids, position_ids, token_type_ids, w):
    """layers/bert_embedding.cpp:24-65 -- word (=), token-type (+=), position (+=), LayerNorm(eps 1e-12)."""
    x = lookup_embedding(w["word"], ids)
    x = lookup_embedding(w["token_type"], token_type_ids, x)
    x = lookup_embedding(w["position"], position_ids, x)
    return layer_norm(x, w["ln_gamma"], w["ln_beta"], 1e-12)


def bert_pooler(x, weight, bias):
    """layers/bert_pooler.cpp:25-37 -- MatMul [B,H]x[H,H] + AddBiasAct<Tanh>."""
    return add_bias_act(mat_mul(x, False, weight, False), bias, "tanh")


def bert_layer(x, ext_mask, lw, num_heads):
    """python/turbo_transformers/layers/modeling_bert.py:238-259 -- attention, intermediate, output."""
    att, _ = multi_headed_attention(x, ext_mask, lw["attention"], num_heads, post_layernorm=True)
    inter = bert_intermediate(att, lw["inter_weight"], lw["inter_bias"])
    return bert_output(inter, att, lw["out_weight"], lw["out_bias"], lw["out_ln_gamma"], lw["out_ln_beta"])


def bert_model(ids, W, num_heads, att_mask=None):
    """python/turbo_transformers/layers/modeling_bert.py:400-434,479-513 -- (sequence_output, pooled_output)."""
    am, tt, pos, ext = prepare_bert_masks(ids, att_mask)
    x = bert_embedding(ids, pos, tt, W["embedding"])
    for lw in W["layers"]:
        x = bert_layer(x, ext, lw, num_heads)
    pooled = bert_pooler(seq_pool(x, "First"), W["pooler_weight"], W["pooler_bias"])
    return x, pooled


def bert_model_smart_batch(id_list, W, num_heads):
    """python/turbo_transformers/layers/modeling_smart_pad.py:434-486,524-559 -- packed [1,sumL,H] output.

    The reference embeds every sequence separately (positions restart at 0) and concatenates.
    """
    seq_list = [len(i) for i in id_list]
    xs = []
    for ids in id_list:
        ids = np.asarray(ids, np.int64)[None]
        _, tt, pos, _ = prepare_bert_masks(ids)
        xs.append(bert_embedding(ids, pos, tt, W["embedding"]))
    x = np.concatenate(xs, 1)
    for lw in W["layers"]:
        att, _ = multi_headed_attention_smart_batch(x, seq_list, lw["attention"], num_heads)
        inter = bert_intermediate(att, lw["inter_weight"], lw["inter_bias"])
        x = bert_output(inter, att, lw["out_weight"], lw["out_bias"], lw["out_ln_gamma"], lw["out_ln_beta"])
    return x


# --------------------------------------------------------------------------------------------------
# Q1: int8 scheme of the benchmark's int8 configuration
# --------------------------------------------------------------------------------------------------
def q_quantize_weight(w):
    """Per-tensor symmetric int8: scale = max|W|/127, q = clip(rint(W/scale), -127, 127)."""
    scale = F32(np.abs(w).max()) / F32(127.0)
    q = np.clip(np.rint(w.astype(F32) / scale), -127, 127).astype(np.int8)
    return q, scale


def q_quantize_rows(x):
    """Per-row dynamic symmetric int8 for activations: scale_r = max|x_r|/127 (1.0 for an all-zero row),
    q = clip(rint(x * (1 / scale_r))) with the reciprocal rounded to fp32 first (multiplying by the inverse scale is how
    quantisers are usually written, torch's among them)."""
    x = x.astype(F32)
    amax = np.abs(x).max(-1, keepdims=True)
    scale = np.where(amax > 0, amax / F32(127.0), F32(1.0)).astype(F32)
    inv = (F32(1.0) / scale).astype(F32)
    q = np.clip(np.rint((x * inv).astype(F32)), -127, 127).astype(np.int8)
    return q, scale


def q_linear(x, wq, w_scale, bias):
    """int8 x int8 -> int32 accumulate, then acc * s_row * s_w + bias (fp32 here; the GPU epilogue rounds to fp16)."""
    xq, xs = q_quantize_rows(x.reshape(-1, x.shape[-1]))
    # products of int8 values summed over K < 2^53 / 127^2 are exact in float64, and float64 has a BLAS behind it
    acc = np.rint(xq.astype(np.float64) @ wq.astype(np.float64)).astype(np.int32)
    return (acc.astype(F32) * xs * F32(w_scale) + bias.astype(F32)).astype(F32)


def q_bert_model(ids, W, num_heads, quantize_attention=True, att_mask=None):
    """BERT forward with the benchmark's int8 scheme on the Linears (all six, or only the two feed-forward
    ones as the reference's qmodeling_bert.py:13-45 did); attention, softmax and layer norms in fp32."""
    def qlin(x, w, b):
        wq, ws = q_quantize_weight(w)
        return q_linear(x, wq, ws, b)

    def flin(x, w, b):
        return mat_mul(x, False, w, False) + b

    _, tt, pos, ext = prepare_bert_masks(ids, att_mask)
    x = bert_embedding(ids, pos, tt, W["embedding"])
    B, L, H = x.shape
    d = H // num_heads
    alin = qlin if quantize_attention else flin
    for lw in W["layers"]:
        a = lw["attention"]
        qkv = alin(x, a["qkv_weight"], a["qkv_bias"]).reshape(B, L, 3, H)
        q, k, v = split_add_bias_transpose_for_score(qkv, np.zeros(3 * H, F32), num_heads)
        p = apply_mask_and_softmax(batch_mat_mul(q, False, k, True, 1.0 / math.sqrt(float(d))), ext, 1.0)
        ctx = transpose_for_score(batch_mat_mul(p, False, v, False))
        o = alin(ctx, a["dense_weight"], a["dense_bias"]).reshape(B, L, H)
        att = layer_norm(o + x, a["ln_gamma"], a["ln_beta"], 1e-12)
        inter = gelu_tanh(qlin(att, lw["inter_weight"], lw["inter_bias"]))
        out = qlin(inter, lw["out_weight"], lw["out_bias"]).reshape(B, L, H)
        x = layer_norm(out + att, lw["out_ln_gamma"], lw["out_ln_beta"], 1e-12)
    return x


# --------------------------------------------------------------------------------------------------
# Q1, the reference's own recipe: torch dynamic quantisation of the two feed-forward Linears
# (python/turbo_transformers/layers/qmodeling_bert.py:13-45). The arithmetic lives in PyTorch
# (torch.quantization.quantize_dynamic, dtype qint8; the reference's docker image pins pytorch 1.7.0), not in the
# reference tree; it is restated here from PyTorch's published algorithm and pinned against the installed torch's
# quantised Linear (tests/test_oracle_pinning.py) and against tests/golden/qbert_recipe_bert_base_b1_s128.npz.
# --------------------------------------------------------------------------------------------------
def qref_quantize_weight(w):
    """MinMaxObserver(qint8, per_tensor_symmetric): scale = max(|min|, |max|) / 127.5, zero point 0,
    q = clamp(rint(w * (1 / scale)), -128, 127).  w is [in, out]; returns (q int8 [in, out], scale fp32)."""
    w = w.astype(F32)
    amax = max(F32(0.0) - min(w.min(), F32(0.0)), max(w.max(), F32(0.0)))
    scale = max(F32(amax) / F32(127.5), F32(np.finfo(np.float32).eps))
    q = np.clip(np.rint(w * (F32(1.0) / scale)), -128, 127).astype(np.int8)
    return q, F32(scale)


def qref_choose_activation_qparams(xmin, xmax, qmin=0, qmax=127):
    """Dynamic per-tensor affine parameters of the activations: the range is widened to contain zero, the scale is
    (max - min) / (qmax - qmin) in double precision, and the zero point is taken from the end of the range with the
    smaller rounding error, then rounded and clamped. qmax = 127, not 255: the x86 engines run with reduce_range."""
    xmin, xmax = min(float(xmin), 0.0), max(float(xmax), 0.0)
    scale = (xmax - xmin) / float(qmax - qmin)
    if F32(scale) == 0.0 or np.isinf(F32(1.0) / F32(scale)):
        scale = 0.1
    zp_from_min, zp_from_max = qmin - xmin / scale, qmax - xmax / scale
    err_min, err_max = abs(qmin) - abs(xmin / scale), abs(qmax) - abs(xmax / scale)
    zp = zp_from_min if err_min < err_max else zp_from_max
    zp = qmin if zp < qmin else (qmax if zp > qmax else int(np.rint(zp)))
    return F32(scale), int(zp)


def qref_quantize_activations(x):
    """x fp32 [M, K] -> (q in [0, 127] as int32, scale, zero point): q = clamp(rint(zp + x * (1 / scale)))."""
    x = x.astype(F32)
    scale, zp = qref_choose_activation_qparams(x.min(), x.max())
    q = np.clip(np.rint(F32(zp) + x * (F32(1.0) / scale)), 0, 127).astype(np.int32)
    return q, scale, zp


def qref_linear(x, wq, w_scale, bias=None):
    """Dynamically quantised Linear: (sum_k (xq - zp) * wq) * (x_scale * w_scale) [+ bias], integer accumulation."""
    xq, xs, zp = qref_quantize_activations(x.reshape(-1, x.shape[-1]))
    acc = np.rint((xq - zp).astype(np.float64) @ wq.astype(np.float64)).astype(np.int64)
    y = acc.astype(F32) * (F32(xs) * F32(w_scale))
    return (y + bias.astype(F32)).astype(F32) if bias is not None else y.astype(F32)


def qref_bert_model(ids, W, num_heads, att_mask=None):
    """BERT forward with the reference's int8 recipe: fp32 attention (BertAttention), the intermediate and output
    Linears dynamically quantised without bias, bias + GELU and bias + residual + LayerNorm re-applied by the
    reference's fused epilogues (layers/addbias_act.cpp:20-23, addbias_layernorm.cpp:20-24)."""
    _, tt, pos, ext = prepare_bert_masks(ids, att_mask)
    x = bert_embedding(ids, pos, tt, W["embedding"])
    for lw in W["layers"]:
        att, _ = multi_headed_attention(x, ext, lw["attention"], num_heads, post_layernorm=True)
        wq, ws = qref_quantize_weight(lw["inter_weight"])
        inter = add_bias_act(qref_linear(att, wq, ws), lw["inter_bias"], "gelu")
        wq, ws = qref_quantize_weight(lw["out_weight"])
        out = qref_linear(inter, wq, ws).reshape(att.shape)
        x = add_bias_layer_norm(att, lw["out_bias"], lw["out_ln_gamma"], lw["out_ln_beta"], out, 1e-12)
    return x


# --------------------------------------------------------------------------------------------------
# G: GPT-2 block composed from the reference's pre-LN flags
# --------------------------------------------------------------------------------------------------
def causal_mask(B, L, neg=-10000.0):
    """3-D additive mask [B,L,L], 0 on/below the diagonal, `neg` above (softmax.cpp:93-102 takes the 3-D branch)."""
    m = np.triu(np.full((L, L), F32(neg), F32), 1)
    return np.tile(m[None], (B, 1, 1))


def gpt2_block(x, mask, lw, num_heads, eps=1e-5):
    """Pre-LN block: MultiHeadedAttention(pre_layernorm, post_add_input) as composed in
    python/turbo_transformers/layers/modeling_encoder.py:81-91, then a pre-LN FFN with the reference's
    tanh-GELU (activation.cpp:32-55, equal to GPT-2's gelu_new) and a residual add (utils.cpp:134-169)."""
    a, _ = multi_headed_attention(x, mask, lw["attention"], num_heads, pre_layernorm=True, post_add_input=True,
                                  pre_ln_eps=eps)
    hdn = layer_norm(a, lw["ln2_gamma"], lw["ln2_beta"], eps)
    inter = add_bias_act(mat_mul(hdn, False, lw["fc_weight"], False), lw["fc_bias"], "gelu")
    out = mat_mul(inter, False, lw["proj_weight"], False).reshape(a.shape)
    return add_input_bias(out, a, lw["proj_bias"])


def gpt2_model(ids, W, num_heads, eps=1e-5, logits=True):
    """wte[ids] + wpe[pos] -> blocks -> final LN -> hidden . wte^T (mat_mul.cpp:30-118 with b_trans)."""
    B, L = ids.shape
    x = (W["wte"][ids] + W["wpe"][np.arange(L)][None]).astype(F32)
    mask = causal_mask(B, L)
    for lw in W["layers"]:
        x = gpt2_block(x, mask, lw, num_heads, eps)
    x = layer_norm(x, W["lnf_gamma"], W["lnf_beta"], eps)
    if not logits:
        return x, None
    return x, mat_mul(x, False, W["wte"], True).reshape(B, L, -1)
