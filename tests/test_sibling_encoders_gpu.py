"""RoBERTa, DistilBERT and ALBERT composed from the BERT kernels (layers/modeling_{roberta,distillbert,albert}.py) against the
HuggingFace fp32 modules on seeded random-init weights, as the reference's roberta_model_test.py / distill_bert_test.py /
albert_model_test.py do (tolerances there: 1e-3 for RoBERTa, 1e-2 for ALBERT). The kernels use the tanh-form GELU like the
reference; RoBERTa's and DistilBERT's torch modules use erf-GELU, which is where most of the fp32 distance comes from.
"""
import copy

import pytest
import torch

import turbotransformers_b200 as tt
from turbotransformers_b200 import synthetic

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
torch.set_grad_enabled(False)
DT = {"f32": (torch.float32, 2e-3), "f16": (torch.float16, 2e-2)}


def seeded(model, seed):
    synthetic.reinit_(model, seed)
    return model.eval()


def ids_and_mask(vocab, batch, seq, seed, lo=3):
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(lo, vocab, (batch, seq), generator=g)
    lens = torch.randint(seq // 2, seq + 1, (batch, ), generator=g)
    mask = (torch.arange(seq)[None, :] < lens[:, None]).long()
    return ids, mask


def check(got, want, mask, tol):
    keep = mask.bool()
    d = (got.float().cpu()[keep] - want[keep]).abs()
    assert torch.isfinite(d).all() and d.max().item() < tol, d.max().item()


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_roberta_model(dt):
    from transformers.models.roberta.modeling_roberta import RobertaConfig, RobertaModel
    cfg = RobertaConfig(vocab_size=1000, hidden_size=256, num_hidden_layers=3, num_attention_heads=4, intermediate_size=1024,
                        max_position_embeddings=130, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=1e-12)
    hf = seeded(RobertaModel(cfg), 11)
    ids, mask = ids_and_mask(cfg.vocab_size, 3, 50, 1)
    want = hf(ids, attention_mask=mask)
    dtype, tol = DT[dt]
    model = tt.RobertaModel.from_torch(copy.deepcopy(hf).to(DEV).to(dtype), DEV)
    seq, pooled = model(ids.to(DEV), attention_mask=mask.to(DEV))[:2]
    check(seq, want.last_hidden_state, mask, tol)
    assert (pooled.float().cpu() - want.pooler_output).abs().max().item() < tol
    # no mask: every position attends everywhere
    seq2 = model(ids.to(DEV))[0]
    check(seq2, hf(ids).last_hidden_state, torch.ones_like(mask), tol)


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_distilbert_model(dt):
    from transformers.models.distilbert.modeling_distilbert import DistilBertConfig, DistilBertModel
    cfg = DistilBertConfig(vocab_size=1000, dim=256, n_layers=3, n_heads=4, hidden_dim=1024, max_position_embeddings=128, dropout=0.0,
                           attention_dropout=0.0)
    hf = seeded(DistilBertModel(cfg), 12)
    ids, mask = ids_and_mask(cfg.vocab_size, 3, 40, 2)
    want = hf(ids, attention_mask=mask).last_hidden_state
    dtype, tol = DT[dt]
    model = tt.DistilBertModel.from_torch(copy.deepcopy(hf).to(DEV).to(dtype))
    got = model(ids.to(DEV), attention_masks=mask.to(DEV).to(dtype))[0]
    check(got, want, mask, tol)
    # the feed-forward block alone against its torch module (same LayerNorm, tanh-GELU against erf-GELU)
    blk = hf.transformer.layer[0]
    x = torch.randn(2, 9, cfg.dim)
    ffn = tt.DistrillFFN.from_torch(copy.deepcopy(blk.ffn).to(DEV).to(dtype), copy.deepcopy(blk.output_layer_norm).to(DEV).to(dtype))
    y = ffn(x.to(DEV).to(dtype))
    assert (y.float().cpu() - blk.output_layer_norm(blk.ffn(x) + x)).abs().max().item() < tol


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_albert_model(dt):
    from transformers.models.albert.modeling_albert import AlbertConfig, AlbertModel
    cfg = AlbertConfig(vocab_size=1000, embedding_size=64, hidden_size=256, num_hidden_layers=4, num_hidden_groups=2, num_attention_heads=4,
                       intermediate_size=1024, max_position_embeddings=128, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0,
                       layer_norm_eps=1e-12, hidden_act="gelu_new")
    hf = seeded(AlbertModel(cfg), 13)
    ids, mask = ids_and_mask(cfg.vocab_size, 2, 33, 3)
    want = hf(ids, attention_mask=mask)
    dtype, tol = DT[dt]
    model = tt.AlbertModel.from_torch(copy.deepcopy(hf).to(DEV).to(dtype))
    seq, pooled = model(ids.to(DEV), attention_mask=mask.to(DEV))
    check(seq, want.last_hidden_state, mask, tol)
    assert (pooled.float().cpu() - want.pooler_output).abs().max().item() < tol
    # layers are shared inside a group: 4 layers, 2 groups -> two distinct AlbertLayer objects
    assert len(model.encoder.albert_layer_groups) == 2
