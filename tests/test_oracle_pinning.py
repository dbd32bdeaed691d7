"""CPU: pins the numpy restatement (oracle/restate.py) to the reference.

1. against the golden vectors in tests/golden/, which the compiled, unmodified reference CPU code produced
   (tests/golden/make_golden.py);
2. against the literal known answers in the reference's own unit tests;
3. live against oracle/_ref when it is present on this machine;
4. the GPT-2 composition (which the reference does not implement) against HuggingFace fp32.
"""
import os

import numpy as np
import pytest
import torch

from oracle import ref_driver, restate
from turbotransformers_b200 import synthetic

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
torch.set_grad_enabled(False)


def gold(name):
    return np.load(os.path.join(GOLD, name + ".npz"))


def weights(g):
    hf = synthetic.make_hf_bert(str(g["model"]), int(g["seed"]))
    return hf, ref_driver.pack_bert_weights(hf)


@pytest.mark.parametrize("name", ["bert_base_b1_s128", "bert_mini_b3_s50_masked"])
def test_fixed_length_model_matches_golden(name):
    g = gold(name)
    hf, W = weights(g)
    mask = g["att_mask"] if g["att_mask"].size else None
    seq, pooled = restate.bert_model(g["ids"], W, hf.config.num_attention_heads, mask)
    assert np.abs(seq - g["sequence_output"]).max() < 2e-5
    assert np.abs(pooled - g["pooled_output"]).max() < 2e-5


@pytest.mark.parametrize("name", ["bert_base_smart_37_5_64", "bert_mini_smart_4_1", "bert_mini_smart_9_7_13"])
def test_smart_batch_model_matches_golden(name):
    g = gold(name)
    hf, W = weights(g)
    lens = [int(n) for n in g["lens"]]
    ids = np.split(g["ids"], np.cumsum(lens)[:-1])
    out = restate.bert_model_smart_batch(ids, W, hf.config.num_attention_heads)
    assert np.abs(out[0] - g["sequence_output"]).max() < 2e-5
    # packed == every sequence on its own (what the reference's smart-batch tests assert)
    solo = np.concatenate([restate.bert_model(i[None], W, hf.config.num_attention_heads)[0][0] for i in ids])
    assert np.abs(out[0] - solo).max() < 2e-5


def test_layer_classes_match_golden():
    g = gold("bert_mini_layer0_b2_s16")
    hf = synthetic.make_hf_bert(str(g["model"]), int(g["seed"]), num_layers=1)
    W = ref_driver.pack_bert_weights(hf)
    heads = hf.config.num_attention_heads
    _, tt, pos, ext = restate.prepare_bert_masks(g["ids"], g["att_mask"])
    emb = restate.bert_embedding(g["ids"], pos, tt, W["embedding"])
    assert np.abs(emb - g["embedding"]).max() < 1e-5
    lw = W["layers"][0]
    att, probs = restate.multi_headed_attention(emb, ext, lw["attention"], heads, post_layernorm=True)
    assert np.abs(att - g["attention_output"]).max() < 1e-5
    assert np.abs(probs - g["attention_probs"]).max() < 1e-6
    inter = restate.bert_intermediate(att, lw["inter_weight"], lw["inter_bias"])
    assert np.abs(inter - g["intermediate"]).max() < 1e-5
    out = restate.bert_output(inter, att, lw["out_weight"], lw["out_bias"], lw["out_ln_gamma"], lw["out_ln_beta"])
    assert np.abs(out - g["layer_output"]).max() < 1e-5


def test_reference_known_answers():
    # layers/kernels/mat_mul_test.cpp:29-77
    a = np.array([[1, 2], [3, 4]], np.float32)
    b = np.array([[2, 3], [4, 5]], np.float32)
    assert restate.mat_mul(a, False, b, False).reshape(-1).tolist() == [10, 13, 22, 29]
    assert restate.batch_mat_mul(np.stack([a, a]), False, np.stack([b, b]), False).reshape(-1).tolist() == [10, 13, 22, 29] * 2


def test_pad_semantics_equal_unpadded_per_sequence():
    # layers/kernels/transpose_test.cpp:242-377: the pad kernels equal the unpadded ones sequence by sequence
    r = np.random.default_rng(0)
    heads, d, lens = 4, 8, [4, 7, 2]
    H = heads * d
    qkv = r.random((1, sum(lens), 3, H), np.float32).astype(np.float32)
    bias = r.random(3 * H).astype(np.float32)
    q, k, v = restate.split_add_bias_transpose_for_score_pad(qkv, bias, heads, lens)
    s = 0
    for b, n in enumerate(lens):
        q1, k1, v1 = restate.split_add_bias_transpose_for_score(qkv[:, s:s + n], bias, heads)
        assert np.array_equal(q[b, :, :n], q1[0]) and np.array_equal(k[b, :, :n], k1[0]) and np.array_equal(v[b, :, :n], v1[0])
        assert not q[b, :, n:].any()
        s += n
    back = restate.transpose_for_score_pad(q, lens)
    assert back.shape == (1, sum(lens), H)
    assert np.array_equal(back[0, :4], restate.transpose_for_score(q[:1, :, :4])[0])


def test_qbert_scheme_vs_reference_recipe_golden():
    """The benchmark's int8 scheme (all six Linears, per-row activations) against the reference's recipe
    (two Linears, torch per-tensor activations): different quantisers, so only closeness is expected."""
    g = gold("qbert_recipe_bert_base_b1_s128")
    hf, W = weights(g)
    heads = hf.config.num_attention_heads
    fp32, _ = restate.bert_model(g["ids"], W, heads)
    recipe_err = np.abs(fp32 - g["sequence_output"])
    # Measured on this fixture: the reference's own int8 recipe is 0.149 max-abs / 0.027 mean-abs away from
    # its fp32 output, so no int8 scheme can be within 5e-2 max-abs of it; the bounds below record reality.
    assert recipe_err.max() < 0.2 and recipe_err.mean() < 0.04
    ours = restate.q_bert_model(g["ids"], W, heads, quantize_attention=False)
    d_fp32, d_recipe = np.abs(ours - fp32), np.abs(ours - g["sequence_output"])
    assert d_fp32.max() < 0.15 and d_fp32.mean() < 0.03          # per-row activation scales: closer to fp32
    assert d_recipe.max() < 0.25 and d_recipe.mean() < 0.045


@pytest.mark.skipif(not ref_driver.available(), reason="oracle/_ref is not built on this machine")
def test_live_reference_agrees_with_restatement():
    hf = synthetic.make_hf_bert("bert-tiny", 7)
    W = ref_driver.pack_bert_weights(hf)
    ids = synthetic.random_ids(2, 24, hf.config.vocab_size, 7)
    ref = ref_driver.RefBert(W, hf.config.num_attention_heads)
    seq, pooled = ref.forward(ids)
    s2, p2 = restate.bert_model(ids.numpy(), W, hf.config.num_attention_heads)
    assert np.abs(seq.numpy() - s2).max() < 1e-5 and np.abs(pooled.numpy() - p2).max() < 1e-5
    idl = synthetic.varlen_ids([5, 16, 9], hf.config.vocab_size, 7)
    sb = ref.forward_smart_batch(idl).numpy()
    sb2 = restate.bert_model_smart_batch([i.numpy() for i in idl], W, hf.config.num_attention_heads)
    assert np.abs(sb - sb2).max() < 1e-5


@pytest.mark.skipif(not ref_driver.available(), reason="oracle/_ref is not built on this machine")
@pytest.mark.parametrize("flags", [(False, False, False), (True, False, True), (False, True, False)])
def test_live_reference_context_attention_agrees_with_restatement(flags):
    pre, post, add = flags
    H, heads, B, Lq, Lk = 64, 4, 2, 5, 9
    w = ref_driver.context_attention_weights(H, 5)
    r = np.random.default_rng(6)
    q = r.standard_normal((B, Lq, H)).astype(np.float32)
    mem = r.standard_normal((B, Lk, H)).astype(np.float32)
    mask = np.zeros((B, 1, Lk), np.float32)
    mask[1, 0, 6:] = -1e18  # the decoder masks the source padding with -1e18
    ref = ref_driver.RefContextAttention(w, heads)
    out, score, kept = ref(q, mem, mem, mask, keep_memory=True, pre_layernorm=pre, post_layernorm=post, post_add_input=add)
    out2, score2, kept2 = restate.context_attention(q, mem, mem, mask, w, heads, None, pre, post, add)
    assert np.abs(out - out2).max() < 1e-5 and np.abs(score - score2).max() < 1e-6
    assert np.abs(kept[0] - kept2[0]).max() < 1e-5 and np.abs(kept[1] - kept2[1]).max() < 1e-5
    # second step: one new query over the kept memory, key / value tensors not consulted
    q1 = r.standard_normal((B, 1, H)).astype(np.float32)
    junk = np.zeros((B, Lk, H), np.float32)
    out_s, _, _ = ref(q1, junk, junk, mask, memory=kept, pre_layernorm=pre, post_layernorm=post, post_add_input=add)
    out_s2, _, _ = restate.context_attention(q1, None, None, mask, w, heads, kept2, pre, post, add)
    assert np.abs(out_s - out_s2).max() < 1e-5


@pytest.mark.skipif(not ref_driver.available(), reason="oracle/_ref is not built on this machine")
def test_live_reference_decoder_layer_agrees_with_restatement():
    H, F, heads, B, Lt, Ls = 64, 160, 4, 2, 6, 9
    lw = ref_driver.decoder_layer_weights(H, F, 3)
    r = np.random.default_rng(4)
    x = r.standard_normal((B, Lt, H)).astype(np.float32)
    mem = r.standard_normal((B, Ls, H)).astype(np.float32)
    src_mask = np.zeros((B, 1, Ls), np.float32)
    src_mask[0, 0, 7:] = -1e18
    dec_mask = (np.triu(np.ones((Lt, Lt), np.float32), 1)[None] * -1e18).repeat(B, 0)
    out, attn = ref_driver.RefDecoderLayer(lw, heads)(x, mem, src_mask, dec_mask)
    out2, attn2, _ = restate.transformer_decoder_layer(x, mem, src_mask, dec_mask, lw, heads)
    assert np.abs(out - out2).max() < 2e-5 and np.abs(attn - attn2).max() < 1e-6


def test_gpt2_composition_matches_huggingface_fp32():
    hf = synthetic.make_hf_gpt2("gpt2-tiny", 3)
    W = ref_driver.pack_gpt2_weights(hf)
    ids = synthetic.random_ids(2, 40, hf.config.vocab_size, 3)
    want = hf(ids).last_hidden_state.numpy()
    got, logits = restate.gpt2_model(ids.numpy(), W, hf.config.n_head)
    assert np.abs(got - want).max() < 2e-4
    assert np.abs(logits - want @ W["wte"].T).max() < 1e-3


def test_int8_restatement_properties():
    r = np.random.default_rng(1)
    w = r.standard_normal((64, 32)).astype(np.float32)
    q, s = restate.q_quantize_weight(w)
    assert q.dtype == np.int8 and np.abs(q).max() == 127 and np.abs(q * s - w).max() <= s / 2 + 1e-7
    x = r.standard_normal((5, 64)).astype(np.float32)
    x[3] = 0
    xq, xs = restate.q_quantize_rows(x)
    assert (np.abs(xq).max(-1)[[0, 1, 2, 4]] == 127).all() and not xq[3].any() and xs[3, 0] == 1.0
    y = restate.q_linear(x, q, s, np.zeros(32, np.float32))
    assert np.abs(y - x @ w).max() < 0.2


def test_reference_int8_recipe_restatement_matches_torch_quantised_linear():
    """qref_*: torch.quantization.quantize_dynamic's arithmetic (the third-party code the reference's recipe calls at
    qmodeling_bert.py:17-18,35-36) restated in numpy, against the installed torch's quantised Linear."""
    import warnings
    torch.manual_seed(0)
    lin = torch.nn.Linear(768, 3072)
    torch.nn.init.normal_(lin.weight, std=0.02)
    torch.nn.init.normal_(lin.bias, std=0.02)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        q = torch.quantization.quantize_dynamic(torch.nn.Sequential(lin), {torch.nn.Linear}, dtype=torch.qint8)[0]
    wt, bias = q._weight_bias()
    wq, ws = restate.qref_quantize_weight(lin.weight.detach().numpy().T.copy())
    assert float(ws) == float(np.float32(wt.q_scale())) and wt.q_zero_point() == 0
    assert np.array_equal(wq.T, wt.int_repr().numpy())
    x = torch.randn(128, 768)
    x[3, 5] = 7.5
    with torch.no_grad():
        want = q(x).numpy()
    got = restate.qref_linear(x.numpy(), wq, ws, bias.detach().numpy())
    assert np.abs(got - want).max() < 2e-6


@pytest.mark.skipif(not ref_driver.available(), reason="oracle/_ref is not built on this machine")
def test_reference_int8_recipe_restatement_layer_by_layer_and_its_amplification():
    """The restated recipe against the live one (torch quantised Linears + the compiled reference's attention and fused
    epilogues), every layer on the live recipe's own input. Then the fact that limits any end-to-end bound: the recipe
    amplifies differences. Layer 0 agrees to fp32 rounding; fed forward through the restatement's own outputs, those 1e-7
    differences flip 7-bit activation roundings and grow to the size of the quantisation noise itself after twelve layers,
    so two faithful implementations of the recipe differ end to end by as much as either differs from fp32."""
    g = gold("qbert_recipe_bert_base_b1_s128")
    hf, W = weights(g)
    heads = hf.config.num_attention_heads
    recipe = ref_driver.RefQBertRecipe(hf)
    h, ext = recipe.embed(g["ids"])
    _, _, _, ext_np = restate.prepare_bert_masks(g["ids"], None)
    worst = 0.0
    for i, lw in enumerate(W["layers"]):
        want = recipe.layer(i, h, ext).numpy()
        x = h.numpy()
        att, _ = restate.multi_headed_attention(x, ext_np, lw["attention"], heads, post_layernorm=True)
        wq, ws = restate.qref_quantize_weight(lw["inter_weight"])
        inter = restate.add_bias_act(restate.qref_linear(att, wq, ws), lw["inter_bias"], "gelu")
        wq, ws = restate.qref_quantize_weight(lw["out_weight"])
        out = restate.qref_linear(inter, wq, ws).reshape(att.shape)
        got = restate.add_bias_layer_norm(att, lw["out_bias"], lw["out_ln_gamma"], lw["out_ln_beta"], out, 1e-12)
        d = float(np.abs(got - want).max())
        if i == 0:
            assert d < 1e-5
        worst = max(worst, d)
        h = torch.from_numpy(want)
    assert worst < 2e-2           # one layer at a time: a handful of flipped roundings at most
    assert np.abs(h.numpy() - g["sequence_output"]).max() < 0.25   # zero on the CPU the golden was made on; elsewhere last-bit BLAS differences get amplified
    free = restate.qref_bert_model(g["ids"], W, heads)
    d = np.abs(free - g["sequence_output"])
    assert 2e-2 < d.max() < 0.25 and d.mean() < 0.04   # measured 0.12 / 0.022: free-running, the restatement drifts that far
