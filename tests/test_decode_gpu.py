"""Decoder step over a key/value cache (ttb_kv_cache_append, ttb_attention_decode, MultiHeadedAttention with layer_cache,
GPT2Model with `past`): the kernel against a numpy softmax over the cache, the cache contents bit-exactly, and the model
through the property that decoding token by token gives what the full-sequence forward gives (checked against the composed
numpy oracle as well). The reference's own check of this path is decoder step vs. full run in its ONMT tests; it has no GPT-2.
"""
import numpy as np
import pytest
import torch

import turbotransformers_b200 as tt
from oracle import ref_driver, restate
from tests.helpers import TORCH_DT, code, host, rng, rounded
from turbotransformers_b200 import _capi, synthetic

pytestmark = pytest.mark.gpu
torch.set_grad_enabled(False)
DEV = torch.device("cuda:0")


def paged(x, B, H):
    """[T, B, H] numpy -> the cache layout [pages, B, 16, H] (zero-filled tail)."""
    T = x.shape[0]
    pages = (T + 15) // 16
    full = np.zeros((pages * 16, B, H), x.dtype)
    full[:T] = x
    return np.ascontiguousarray(full.reshape(pages, 16, B, H).transpose(0, 2, 1, 3))


def unpaged(p, T):
    pages, B, _, H = p.shape
    return p.transpose(0, 2, 1, 3).reshape(pages * 16, B, H)[:T]


def decode_oracle(qkv, k_cache, v_cache, B, n_new, heads, past, scale):
    """Row b*n_new+t of qkv attends cache rows 0..past+t of sequence b (the new rows already appended)."""
    H = heads * 64
    out = np.zeros((B * n_new, H), np.float32)
    for b in range(B):
        for t in range(n_new):
            q = qkv[b * n_new + t, :H].reshape(heads, 64)
            n = past + t + 1
            K = k_cache[:n, b].reshape(n, heads, 64)
            V = v_cache[:n, b].reshape(n, heads, 64)
            s = np.einsum("hd,nhd->hn", q, K) * scale
            p = np.exp(s - s.max(1, keepdims=True))
            p /= p.sum(1, keepdims=True)
            out[b * n_new + t] = np.einsum("hn,nhd->hd", p, V).reshape(H)
    return out


@pytest.mark.parametrize("dt", ["f16", "bf16"])
@pytest.mark.parametrize("B,heads,past,n_new", [(1, 2, 0, 1), (3, 12, 5, 1), (2, 4, 130, 3), (4, 12, 1000, 1), (1, 12, 63, 17)])
def test_attention_decode_matches_numpy(ctx, dt, B, heads, past, n_new):
    r = rng(B * 1000 + past + n_new)
    H = heads * 64
    cap = past + n_new + 3
    qkv = rounded(r.standard_normal((B * n_new, 3 * H)).astype(np.float32), dt)
    kc = rounded(r.standard_normal((cap, B, H)).astype(np.float32), dt)
    vc = rounded(r.standard_normal((cap, B, H)).astype(np.float32), dt)
    Kc, Vc = torch.from_numpy(paged(kc, B, H)).to(DEV).to(TORCH_DT[dt]), torch.from_numpy(paged(vc, B, H)).to(DEV).to(TORCH_DT[dt])
    Q = torch.from_numpy(qkv).to(DEV).to(TORCH_DT[dt])
    out = torch.full((B * n_new, H), float("nan"), dtype=TORCH_DT[dt], device=DEV)
    ctx.call("attention_decode", code(dt), Q, B, n_new, heads, 64, Kc, Vc, past, 0.125, out)
    assert ctx.device_status() == _capi.OK
    # the new keys / values sit in rows [past, past + n_new), everything else is untouched
    want_k, want_v = kc.copy(), vc.copy()
    for b in range(B):
        for t in range(n_new):
            want_k[past + t, b] = qkv[b * n_new + t, H:2 * H]
            want_v[past + t, b] = qkv[b * n_new + t, 2 * H:]
    assert np.array_equal(unpaged(host(Kc), cap), want_k) and np.array_equal(unpaged(host(Vc), cap), want_v)
    want = decode_oracle(qkv, want_k, want_v, B, n_new, heads, past, 0.125)
    tol = 4e-3 if dt == "f16" else 3e-2
    assert np.abs(host(out) - want).max() < tol
    # the stand-alone append writes the same rows
    Kc2, Vc2 = torch.from_numpy(paged(kc, B, H)).to(DEV).to(TORCH_DT[dt]), torch.from_numpy(paged(vc, B, H)).to(DEV).to(TORCH_DT[dt])
    ctx.call("kv_cache_append", code(dt), Q, B, n_new, heads, 64, Kc2, Vc2, past)
    assert torch.equal(Kc2, Kc) and torch.equal(Vc2, Vc)


def test_attention_decode_rejects_bad_arguments(ctx):
    t = torch.zeros(8, 3 * 128, dtype=torch.float16, device=DEV)
    c = torch.zeros(1, 1, 16, 128, dtype=torch.float16, device=DEV)
    o = torch.zeros(8, 128, dtype=torch.float16, device=DEV)
    import ctypes as C
    lib = _capi.lib()
    P = lambda x: C.c_void_p(x.data_ptr())
    assert lib.ttb_attention_decode(ctx.h, _capi.F32, P(t), 1, 1, 2, 64, P(c), P(c), 0, 0.125, P(o)) == _capi.ERR_INVALID  # dtype
    assert lib.ttb_attention_decode(ctx.h, _capi.F16, P(t), 1, 1, 4, 32, P(c), P(c), 0, 0.125, P(o)) == _capi.ERR_INVALID  # head size
    assert lib.ttb_attention_decode(ctx.h, _capi.F16, P(t), 1, 65, 2, 64, P(c), P(c), 0, 0.125, P(o)) == _capi.ERR_INVALID  # too many new tokens


@pytest.mark.parametrize("dt", ["f16", "bf16"])
def test_gpt2_incremental_decoding_equals_full_forward(dt):
    hf32 = synthetic.make_hf_gpt2("gpt2-mini", 5)
    W = ref_driver.pack_gpt2_weights(hf32)
    B, L0, steps = 3, 17, 9
    L = L0 + steps + 3
    ids = synthetic.random_ids(B, L, hf32.config.vocab_size, 2)
    want, want_logits = restate.gpt2_model(ids.numpy(), W, hf32.config.n_head)
    model = tt.GPT2Model.from_torch(hf32.to(DEV).to(TORCH_DT[dt]), DEV)
    full, full_logits = model(ids.to(DEV))
    past = model.new_cache()
    pieces, logit_pieces = [], []
    h, lg = model(ids[:, :L0].to(DEV), past=past)  # prompt
    pieces.append(h)
    logit_pieces.append(lg)
    for s in range(steps):  # one token at a time
        h, lg = model(ids[:, L0 + s:L0 + s + 1].contiguous().to(DEV), past=past)
        pieces.append(h)
        logit_pieces.append(lg)
        assert model.cached_length(past) == L0 + s + 1
    h, lg = model(ids[:, L0 + steps:].contiguous().to(DEV), past=past)  # three tokens at once
    pieces.append(h)
    logit_pieces.append(lg)
    inc = torch.cat(pieces, 1).float().cpu().numpy()
    inc_logits = torch.cat(logit_pieces, 1).float().cpu().numpy()
    tol, mean_tol = (2e-2, 2e-3) if dt == "f16" else (1.6e-1, 1.6e-2)
    d_full = np.abs(inc - full.float().cpu().numpy())
    assert d_full.max() < tol and d_full.mean() < mean_tol  # cached decoding == full-sequence forward
    d = np.abs(inc - want)
    assert d.max() < tol and d.mean() < mean_tol            # and == the composed fp32 oracle
    assert np.abs(inc_logits - want_logits).max() < tol * 4


def test_gpt2_token_by_token_from_the_first_token():
    hf32 = synthetic.make_hf_gpt2("gpt2-tiny", 1, num_layers=1)
    model = tt.GPT2Model.from_torch(hf32.to(DEV).half(), DEV)
    B, L = 2, 120
    ids = synthetic.random_ids(B, L, hf32.config.vocab_size, 3)
    full = model(ids.to(DEV), return_logits=False)[0].float().cpu().numpy()
    past = model.new_cache()
    out = [model(ids[:, :1].to(DEV), return_logits=False, past=past)[0]]
    for s in range(1, L):
        out.append(model(ids[:, s:s + 1].contiguous().to(DEV), return_logits=False, past=past)[0])
    inc = torch.cat(out, 1).float().cpu().numpy()
    assert model.cached_length(past) == L
    assert np.abs(inc - full).max() < 2e-2
    with pytest.raises(NotImplementedError):
        tt.GPT2Model.from_torch(synthetic.make_hf_gpt2("gpt2-tiny", 1).to(DEV), DEV).new_cache()  # fp32 has no cached path
