"""TransformerDecoderLayer / TransformerDecoder (the OpenNMT-py style decoder of the reference's modeling_decoder.py) against
the numpy restatement of the reference's composition, which tests/test_oracle_pinning.py pins to the compiled reference.

Tolerances (max-abs, outputs of order one): fp32 2e-4; fp16 3e-2 after three sub-blocks with activations kept in fp16.
Stepwise decoding (16-bit) must reproduce, token by token, the full-sequence pass under the future mask.
"""
import numpy as np
import pytest
import torch

import turbotransformers_b200 as tt
from oracle import ref_driver, restate
from tests.helpers import TORCH_DT, rounded

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
torch.set_grad_enabled(False)


def linear(w_in_out, bias):
    lin = torch.nn.Linear(w_in_out.shape[0], w_in_out.shape[1])
    lin.weight.copy_(torch.from_numpy(w_in_out).t())
    lin.bias.copy_(torch.from_numpy(bias))
    return lin


def norm(gamma, beta, eps):
    ln = torch.nn.LayerNorm(gamma.shape[0], eps=eps)
    ln.weight.copy_(torch.from_numpy(gamma))
    ln.bias.copy_(torch.from_numpy(beta))
    return ln


class OnmtStyleAttention(torch.nn.Module):
    def __init__(self, w, heads):
        super().__init__()
        self.head_count, self.max_relative_positions = heads, 0
        self.linear_keys, self.linear_values = linear(w["k_weight"], w["k_bias"]), linear(w["v_weight"], w["v_bias"])
        self.linear_query, self.final_linear = linear(w["q_weight"], w["q_bias"]), linear(w["dense_weight"], w["dense_bias"])


class OnmtStyleFFN(torch.nn.Module):
    def __init__(self, f):
        super().__init__()
        self.w_1, self.w_2 = linear(f["w1_weight"], f["w1_bias"]), linear(f["w2_weight"], f["w2_bias"])
        self.layer_norm = norm(f["ln_gamma"], f["ln_beta"], 1e-12)  # the epsilon the reference's FFN hard-codes


class OnmtStyleDecoderLayer(torch.nn.Module):
    def __init__(self, lw, heads):
        super().__init__()
        self.self_attn = OnmtStyleAttention(lw["self"]["split"], heads)
        self.context_attn = OnmtStyleAttention(lw["context"], heads)
        self.feed_forward = OnmtStyleFFN(lw["ffn"])
        self.layer_norm_1 = norm(lw["self"]["ln_gamma"], lw["self"]["ln_beta"], 1e-6)
        self.layer_norm_2 = norm(lw["context"]["ln_gamma"], lw["context"]["ln_beta"], 1e-6)


def round_weights(lw, dt):
    def rw(d):
        return {k: (rw(v) if isinstance(v, dict) else rounded(v, dt)) for k, v in d.items()}
    return rw(lw)


def diff(t, want):
    return float(np.abs(t.detach().float().cpu().numpy().reshape(want.shape) - want).max())


@pytest.mark.parametrize("dt,tol", [("f32", 2e-4), ("f16", 3e-2)])
def test_decoder_layer_full_sequence_matches_restatement(dt, tol):
    H, F, heads, B, Lt, Ls = 768, 1024, 12, 2, 9, 21
    lw = round_weights(ref_driver.decoder_layer_weights(H, F, 21), dt)
    r = np.random.default_rng(22)
    x = rounded(r.standard_normal((B, Lt, H)).astype(np.float32), dt)
    mem = rounded(r.standard_normal((B, Ls, H)).astype(np.float32), dt)
    src_pad = np.zeros((B, 1, Ls), bool)
    src_pad[1, 0, 15:] = True
    tgt_pad = np.zeros((B, 1, Lt), bool)
    tgt_pad[0, 0, 7:] = True
    dec_mask = ((tgt_pad.astype(np.float32) + np.triu(np.ones((Lt, Lt), np.float32), 1)[None]) > 0).astype(np.float32) * np.float32(-1e18)
    want, want_attn, _ = restate.transformer_decoder_layer(x, mem, src_pad.astype(np.float32) * np.float32(-1e18), dec_mask, lw, heads)
    layer = tt.TransformerDecoderLayer.from_onmt(OnmtStyleDecoderLayer(lw, heads).to(DEV).to(TORCH_DT[dt]))
    X, M = torch.from_numpy(x).to(DEV).to(TORCH_DT[dt]), torch.from_numpy(mem).to(DEV).to(TORCH_DT[dt])
    out, attn, align = layer(X, M, torch.from_numpy(src_pad).to(DEV), torch.from_numpy(tgt_pad).to(DEV))
    assert align is None and out.dtype == TORCH_DT[dt] and tuple(attn.shape) == (B, Lt, Ls)
    keep = ~tgt_pad[:, 0]  # rows of padded target positions are not defined by the model
    assert diff(out[torch.from_numpy(keep).to(DEV)], want[keep]) < tol
    assert diff(attn[torch.from_numpy(keep).to(DEV)], want_attn[keep]) < tol
    assert tt._cxx_module.device_status(0) == 0


def test_stepwise_decoding_reproduces_the_full_sequence_pass_fp16():
    H, F, heads, B, Lt, Ls, n_layers = 768, 1024, 12, 3, 6, 17, 2
    r = np.random.default_rng(31)
    lws = [round_weights(ref_driver.decoder_layer_weights(H, F, 40 + i), "f16") for i in range(n_layers)]
    layers = [tt.TransformerDecoderLayer.from_onmt(OnmtStyleDecoderLayer(lw, heads).to(DEV).half()) for lw in lws]
    x = torch.from_numpy(r.standard_normal((B, Lt, H)).astype(np.float32)).to(DEV).half()
    mem = torch.from_numpy(r.standard_normal((B, Ls, H)).astype(np.float32)).to(DEV).half()
    src_pad = torch.zeros(B, 1, Ls, dtype=torch.bool, device=DEV)
    src_pad[2, 0, 11:] = True
    tgt_pad = torch.zeros(B, 1, Lt, dtype=torch.bool, device=DEV)
    full = x
    for layer in layers:
        full, full_attn, _ = layer(full, mem, src_pad, tgt_pad)
    caches = [{"memory_keys": None, "memory_values": None, "self_keys": None, "self_values": None} for _ in layers]
    for t in range(Lt):
        h = x[:, t:t + 1].contiguous()
        for layer, cache in zip(layers, caches):
            h, attn, _ = layer(h, mem, src_pad, tgt_pad[:, :, t:t + 1], layer_cache=cache, step=t)
        # the pre-LN residual stream is not normalised: its values reach ten and more, where an fp16 step is 0.008, and the
        # one-token GEMMs (split along K over a cluster) round in another order than the full-sequence ones
        assert (h[:, 0].float() - full[:, t].float()).abs().max().item() < 4e-2, t
        assert (attn[:, 0].float() - full_attn[:, t].float()).abs().max().item() < 1e-2
    assert tuple(caches[0]["memory_keys"].shape) == (B, heads, Ls, H // heads)
    assert caches[0]["self_keys"].shape(0) == Lt  # the in-place cache holds every decoded position
    assert tt._cxx_module.device_status(0) == 0


class Embeddings(torch.nn.Module):
    """Token embedding with OpenNMT-py's call signature: [len, B, 1] ids -> [len, B, H]."""
    word_padding_idx = 1

    def __init__(self, vocab, H):
        super().__init__()
        self.table = torch.nn.Embedding(vocab, H)

    def forward(self, tgt, step=None):
        return self.table(tgt[:, :, 0])


def test_transformer_decoder_stack_fp32_matches_restatement():
    H, F, heads, B, Lt, Ls, n_layers, vocab = 128, 256, 2, 2, 5, 8, 2, 50

    class Stack(torch.nn.Module):
        def __init__(self, lws):
            super().__init__()
            self.embeddings = Embeddings(vocab, H)
            self.transformer_layers = torch.nn.ModuleList([OnmtStyleDecoderLayer(lw, heads) for lw in lws])
            self.layer_norm = torch.nn.LayerNorm(H, eps=1e-6)
            self._copy, self.alignment_layer = False, 0

    lws = [ref_driver.decoder_layer_weights(H, F, 60 + i) for i in range(n_layers)]
    torch.manual_seed(0)
    stack = Stack(lws).to(DEV)
    dec = tt.TransformerDecoder.from_onmt(stack, DEV)
    tgt = torch.randint(2, vocab, (Lt, B, 1), device=DEV)
    tgt[4, 1, 0] = Embeddings.word_padding_idx
    memory_bank = torch.randn(Ls, B, H, device=DEV)
    lengths = torch.tensor([Ls, 5], device=DEV)
    dec.init_state(torch.zeros(Ls, B, 1), memory_bank, None)
    outs, attns = dec(tgt, memory_bank, memory_lengths=lengths)
    assert tuple(outs.shape) == (Lt, B, H) and tuple(attns["std"].shape) == (Lt, B, Ls)
    # the same pass through the restatement
    x = stack.embeddings(tgt).transpose(0, 1).cpu().numpy()
    mem = memory_bank.transpose(0, 1).contiguous().cpu().numpy()
    src_mask = np.zeros((B, 1, Ls), np.float32)
    src_mask[1, 0, 5:] = -1e18
    tgt_pad = (tgt[:, :, 0].t() == 1).cpu().numpy().astype(np.float32)[:, None]
    dec_mask = ((tgt_pad + np.triu(np.ones((Lt, Lt), np.float32), 1)[None]) > 0).astype(np.float32) * np.float32(-1e18)
    for lw in lws:
        x, attn, _ = restate.transformer_decoder_layer(x, mem, src_mask, dec_mask, lw, heads)
    want = restate.layer_norm(x, stack.layer_norm.weight.cpu().numpy(), stack.layer_norm.bias.cpu().numpy(), 1e-6)
    keep = tgt_pad[:, 0] == 0
    got = outs.transpose(0, 1).cpu().numpy()
    assert np.abs(got[keep] - want[keep]).max() < 2e-4
    assert np.abs(attns["std"].transpose(0, 1).cpu().numpy()[keep] - attn[keep]).max() < 1e-4
