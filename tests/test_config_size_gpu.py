"""Parity at the sizes the benchmark configurations name, against the compiled reference CPU code (oracle/_ref) where it
has the model and against the numpy restatement otherwise. Batch elements are independent, so where the CPU oracle would
take minutes for a whole batch the GPU runs the full batch and the oracle a leading sub-batch.

  config 2 sweep corners : BERT-base fp16, 32 x 32 and 8 x 512
  config 3               : BERT-base int8 (all six Linears), 16 x 128
  config 4               : BERT-large fp16, all 24 layers, 2 x 512
  config 5               : GPT-2 small fp16, all 12 layers, 1 x 1024, hidden states and the 50257-wide logits

Tolerances: 2e-2 max-abs / 2e-3 mean-abs on final hidden states for 16-bit models; int8 against the integer oracle of
the same scheme as in test_model_gpu.py.
"""
import numpy as np
import pytest
import torch

import turbotransformers_b200 as tt
from oracle import ref_driver, restate
from turbotransformers_b200 import synthetic

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
torch.set_grad_enabled(False)
MAX_TOL, MEAN_TOL = 2e-2, 2e-3


def close(got, want, max_tol=MAX_TOL, mean_tol=MEAN_TOL):
    d = np.abs(got.detach().float().cpu().numpy().reshape(want.shape) - want)
    assert np.isfinite(d).all()
    assert d.max() < max_tol, f"max-abs {d.max():.4g}"
    assert d.mean() < mean_tol, f"mean-abs {d.mean():.4g}"


def oracle_bert(W, heads, ids):
    """(sequence_output, pooled_output) of the reference for int64 ids [b, L]."""
    if ref_driver.available():
        seq, pooled = ref_driver.RefBert(W, heads).forward(ids)
        return seq.numpy(), pooled.numpy()
    return restate.bert_model(ids.numpy(), W, heads)


@pytest.mark.parametrize("batch,seq_len,sub", [(32, 32, 32), (8, 512, 2)])
def test_bert_base_fp16_sweep_corners(batch, seq_len, sub):
    hf32 = synthetic.make_hf_bert("bert-base", 0)
    ids = synthetic.random_ids(batch, seq_len, hf32.config.vocab_size, 7)
    W = ref_driver.pack_bert_weights(hf32)
    want, want_pooled = oracle_bert(W, 12, ids[:sub])
    model = tt.BertModel.from_torch(hf32.to(DEV).half(), DEV)
    seq, pooled = model(ids.to(DEV))[:2]
    assert tuple(seq.shape) == (batch, seq_len, 768)
    close(seq[:sub], want)
    close(pooled[:sub], want_pooled)
    assert tt._cxx_module.device_status(0) == 0


def test_bert_large_full_depth_fp16():
    hf32 = synthetic.make_hf_bert("bert-large", 0)
    assert hf32.config.num_hidden_layers == 24 and hf32.config.hidden_size == 1024
    ids = synthetic.random_ids(2, 512, hf32.config.vocab_size, 0)
    W = ref_driver.pack_bert_weights(hf32)
    want, want_pooled = oracle_bert(W, 16, ids)
    model = tt.BertModel.from_torch(hf32.to(DEV).half(), DEV)
    seq, pooled = model(ids.to(DEV))[:2]
    close(seq, want)
    close(pooled, want_pooled)
    assert tt._cxx_module.device_status(0) == 0


def test_gpt2_small_full_size_fp16():
    hf32 = synthetic.make_hf_gpt2("gpt2-small", 0)
    cfg = hf32.config
    assert cfg.n_layer == 12 and cfg.vocab_size == 50257 and cfg.n_positions >= 1024
    ids = synthetic.random_ids(1, 1024, cfg.vocab_size, 0)
    W = ref_driver.pack_gpt2_weights(hf32)
    want, want_logits = restate.gpt2_model(ids.numpy(), W, cfg.n_head)
    model = tt.GPT2Model.from_torch(hf32.to(DEV).half(), DEV)
    hidden, logits = model(ids.to(DEV))
    assert tuple(logits.shape) == (1, 1024, 50257)
    close(hidden, want)
    close(logits, want_logits)
    assert tt._cxx_module.device_status(0) == 0


def test_qbert_b16_s128_against_integer_oracle():
    hf32 = synthetic.make_hf_bert("bert-base", 0)
    ids = synthetic.random_ids(16, 128, hf32.config.vocab_size, 11)
    W = ref_driver.pack_bert_weights(hf32)
    sub = 4
    want = restate.q_bert_model(ids[:sub].numpy(), W, 12, True)
    model = tt.QBertModel.from_torch(hf32.to(DEV).half(), DEV)
    seq = model(ids.to(DEV))[0]
    assert tuple(seq.shape) == (16, 128, 768)
    # same bounds as the b1 case in test_model_gpu.py: sixteen-bit activations between layers move some values across an
    # int8 rounding boundary, which twelve layers amplify
    close(seq[:sub], want, 0.15, 2.5e-2)
    assert tt._cxx_module.device_status(0) == 0
