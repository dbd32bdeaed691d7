"""Context (encoder-decoder) attention of MultiHeadedAttention against the numpy restatement of the reference's context branch
(layers/multi_headed_attention.cpp:45-167,260-380), which tests/test_oracle_pinning.py pins to the compiled reference.

Tolerances (max-abs, outputs of order one): fp32 1e-4, fp16 1e-2, bf16 6e-2; the 16-bit paths keep activations in the
storage type between the reference's ops.
"""
import numpy as np
import pytest
import torch

import turbotransformers_b200 as tt
from oracle import ref_driver, restate
from tests.helpers import TORCH_DT, rounded

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
TOL = {"f32": 1e-4, "f16": 1e-2, "bf16": 6e-2}
torch.set_grad_enabled(False)


class OnmtStyleAttention(torch.nn.Module):
    """Parameter names and attributes of OpenNMT-py's MultiHeadedAttention (what from_onmt reads)."""

    def __init__(self, w, heads):
        super().__init__()
        H = w["q_weight"].shape[0]
        self.head_count, self.max_relative_positions = heads, 0
        for name, key in (("linear_keys", "k"), ("linear_values", "v"), ("linear_query", "q"), ("final_linear", "dense")):
            lin = torch.nn.Linear(H, H)
            lin.weight.copy_(torch.from_numpy(w[key + "_weight"]).t())
            lin.bias.copy_(torch.from_numpy(w[key + "_bias"]))
            setattr(self, name, lin)


def build(w, heads, dt):
    mod = OnmtStyleAttention(w, heads).to(DEV).to(TORCH_DT[dt])
    ln = torch.nn.LayerNorm(w["ln_gamma"].shape[0])
    ln.weight.copy_(torch.from_numpy(w["ln_gamma"]))
    ln.bias.copy_(torch.from_numpy(w["ln_beta"]))
    return tt.MultiHeadedAttention.from_onmt(mod, ln.to(DEV).to(TORCH_DT[dt]))


def on_dev(a, dt):
    return torch.from_numpy(a).to(DEV).to(TORCH_DT[dt])


def diff(t, want):
    return float(np.abs(t.detach().float().cpu().numpy().reshape(want.shape) - want).max())


@pytest.mark.parametrize("dt", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("flags", [(False, False, False), (True, False, True), (False, True, False)])
def test_context_attention_matches_restatement_with_and_without_memory_cache(dt, flags):
    pre, post, add = flags
    H, heads, B, Lq, Lk = 768, 12, 3, 7, 37
    w = {k: rounded(v, dt) for k, v in ref_driver.context_attention_weights(H, 11).items()}
    r = np.random.default_rng(12)
    q = rounded(r.standard_normal((B, Lq, H)).astype(np.float32), dt)
    mem = rounded(r.standard_normal((B, Lk, H)).astype(np.float32), dt)
    mask = np.zeros((B, 1, Lk), np.float32)
    mask[1, 0, 20:] = -1e18
    mask[2, 0, 5:] = -1e18
    want, want_prob, want_mem = restate.context_attention(q, mem, mem, mask, w, heads, None, pre, post, add)
    att = build(w, heads, dt)
    kw = dict(attn_type="context", pre_layernorm=pre, post_layernorm=post, post_add_input=add)
    Q, M, MASK = on_dev(q, dt), on_dev(mem, dt), torch.from_numpy(mask).to(DEV)

    out, prob = att(M, M, Q, mask=MASK, **kw)  # no cache
    assert out.dtype == TORCH_DT[dt] and tuple(out.shape) == (B, Lq, H)
    assert diff(out, want) < TOL[dt]
    prob = torch.utils.dlpack.from_dlpack(prob.to_dlpack())
    assert tuple(prob.shape) == (B, heads, Lq, Lk) and diff(prob, want_prob) < TOL[dt] * 0.5
    assert float(prob[1, :, :, 20:].float().abs().max()) == 0.0  # masked source positions get no weight

    cache = {"memory_keys": None, "memory_values": None}  # first step files the projected memory
    out1, _ = att(M, M, Q, mask=MASK, layer_cache=cache, **kw)
    assert diff(out1, want) < TOL[dt]
    assert tuple(cache["memory_keys"].shape) == (B, heads, Lk, H // heads)
    assert diff(cache["memory_keys"], want_mem[0]) < TOL[dt] and diff(cache["memory_values"], want_mem[1]) < TOL[dt]

    q1 = rounded(r.standard_normal((B, 1, H)).astype(np.float32), dt)  # next step: one query over the kept memory
    want_s, _, _ = restate.context_attention(q1, None, None, mask, w, heads, want_mem, pre, post, add)
    junk = torch.zeros(B, Lk, H, device=DEV, dtype=TORCH_DT[dt])
    out_s, _ = att(junk, junk, on_dev(q1, dt), mask=MASK, layer_cache=cache, **kw)
    assert tuple(out_s.shape) == (B, 1, H) and diff(out_s, want_s) < TOL[dt]
    assert tt._cxx_module.device_status(0) == 0


def test_context_attention_per_query_mask_and_error_cases():
    H, heads, B, Lq, Lk = 128, 2, 2, 4, 6
    w = ref_driver.context_attention_weights(H, 13)
    r = np.random.default_rng(14)
    q = r.standard_normal((B, Lq, H)).astype(np.float32)
    mem = r.standard_normal((B, Lk, H)).astype(np.float32)
    mask = np.where(r.random((B, Lq, Lk)) < 0.3, -1e18, 0.0).astype(np.float32)
    mask[:, :, 0] = 0.0
    want, _, _ = restate.context_attention(q, mem, mem, mask, w, heads)
    att = build(w, heads, "f32")
    out, _ = att(on_dev(mem, "f32"), on_dev(mem, "f32"), on_dev(q, "f32"), mask=torch.from_numpy(mask).to(DEV), attn_type="context")
    assert diff(out, want) < 1e-4
    with pytest.raises(Exception, match="memory_keys and memory_values"):
        att(on_dev(mem, "f32"), on_dev(mem, "f32"), on_dev(q, "f32"), attn_type="context", layer_cache={"memory_keys": None})
    with pytest.raises(Exception, match="context or self"):
        att(on_dev(mem, "f32"), on_dev(mem, "f32"), on_dev(q, "f32"), attn_type="cross")
    from turbotransformers_b200 import synthetic
    bert_att = tt.MultiHeadedAttention.from_torch(synthetic.make_hf_bert("bert-tiny", 1).encoder.layer[0].attention.to(DEV))
    x = torch.randn(2, 4, 128, device=DEV)
    with pytest.raises(Exception, match="separate q, k, v"):
        bert_att(x, x, x, attn_type="context")


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("flags", [(False, False, False), (True, False, True), (False, True, False)])
def test_smart_batch_context_attention_with_query_and_key_length_lists(dt, flags):
    """MultiHeadedAttentionSmartBatch with attn_type="context" (multi_headed_attention_smart_batch.cpp:34-170): packed queries
    of lengths [9, 7, 13] against packed keys / values of lengths [10, 19, 20], the lists of the reference's own test
    (python/tests/multi_head_attn_smart_batch_test.py:155-165). As there, the expected result is every sequence run alone
    through the fixed-length attention (here its restatement, pinned to the compiled reference), concatenated."""
    pre, post, add = flags
    H, heads = 768, 12
    q_lens, k_lens = [9, 7, 13], [10, 19, 20]
    w = {k: rounded(v, dt) for k, v in ref_driver.context_attention_weights(H, 21).items()}
    r = np.random.default_rng(22)
    qs = [rounded(r.random((1, n, H)).astype(np.float32), dt) for n in q_lens]
    ks = [rounded(r.random((1, n, H)).astype(np.float32), dt) for n in k_lens]
    vs = [rounded(r.random((1, n, H)).astype(np.float32), dt) for n in k_lens]
    want = np.concatenate([restate.context_attention(q, k, v, None, w, heads, None, pre, post, add)[0] for q, k, v in zip(qs, ks, vs)], 1)
    mod = OnmtStyleAttention(w, heads).to(DEV).to(TORCH_DT[dt])
    ln = torch.nn.LayerNorm(H)
    ln.weight.copy_(torch.from_numpy(w["ln_gamma"]))
    ln.bias.copy_(torch.from_numpy(w["ln_beta"]))
    att = tt.MultiHeadedAttentionSmartBatch.from_onmt(mod, ln.to(DEV).to(TORCH_DT[dt]))
    Q, K, V = (on_dev(np.concatenate(x, 1), dt) for x in (qs, ks, vs))
    kw = dict(attn_type="context", pre_layernorm=pre, post_layernorm=post, post_add_input=add)
    out, prob = att(K, V, Q, q_lens, k_lens, mask=None, **kw)
    assert tuple(out.shape) == (1, sum(q_lens), H)
    assert diff(out, want) < TOL[dt]
    prob = torch.utils.dlpack.from_dlpack(prob.to_dlpack())
    assert tuple(prob.shape) == (3, heads, max(q_lens), max(k_lens))
    assert float(prob[0, :, :9, 10:].float().abs().max()) == 0.0   # keys beyond a sequence's own length get no weight
    # the projected memory can be kept and used again, as in the fixed-length class
    cache = {"memory_keys": None, "memory_values": None}
    out1, _ = att(K, V, Q, q_lens, k_lens, layer_cache=cache, **kw)
    assert diff(out1, want) < TOL[dt] and tuple(cache["memory_keys"].shape) == (3, heads, max(k_lens), H // heads)
    junk = torch.zeros_like(K)
    out2, _ = att(junk, junk, Q, q_lens, k_lens, layer_cache=cache, **kw)
    assert diff(out2, want) < TOL[dt]
    with pytest.raises(Exception, match="batch size"):
        att(K, V, Q, q_lens, k_lens[:2], **kw)
    assert tt._cxx_module.device_status(0) == 0
