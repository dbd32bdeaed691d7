"""Seeded synthetic models and inputs shaped like the benchmark configurations.

The reference benchmarks on random ids and (for speed runs) random-initialised HuggingFace modules
(benchmark/turbo_benchmark_helper.py:68-72); no dataset is involved.  Weights: every Linear and
embedding matrix ~ N(0, 0.02), every Linear bias ~ N(0, 0.02) (non-zero so the bias paths are
exercised), LayerNorm gamma = 1 and beta = 0.  Everything is drawn in fp32 from one
torch.Generator(seed) in named_parameters() order, so the same seed gives the same model on any box;
lower-precision models are made by casting afterwards.
"""
import random

import torch

CONFIGS = {
    # name: (layers, hidden, heads, ffn, vocab, positions, type_vocab)
    "bert-base": (12, 768, 12, 3072, 30522, 512, 2),
    "bert-large": (24, 1024, 16, 4096, 30522, 512, 2),
    "bert-tiny": (2, 128, 2, 512, 1000, 128, 2),
    "bert-mini": (3, 256, 4, 1024, 2000, 512, 2),
}


def bert_config(name="bert-base", num_layers=None):
    from transformers.models.bert.modeling_bert import BertConfig
    n, h, a, f, v, p, t = CONFIGS[name]
    return BertConfig(vocab_size=v, hidden_size=h, num_hidden_layers=num_layers or n, num_attention_heads=a,
                      intermediate_size=f, max_position_embeddings=p, type_vocab_size=t,
                      hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0, layer_norm_eps=1e-12)


def reinit_(module, seed, std=0.02):
    """Overwrite every parameter in place from torch.Generator(seed); LayerNorm -> (1, 0)."""
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in module.named_parameters():
            if "LayerNorm" in name or ".ln_" in name or name.startswith("ln_"):
                p.fill_(1.0 if name.endswith("weight") else 0.0)
            else:
                p.copy_(torch.randn(p.shape, generator=g, dtype=torch.float32) * std)
    return module


def make_hf_bert(name="bert-base", seed=0, num_layers=None):
    """A HuggingFace BertModel (fp32, eval, CPU) with the seeded weights described above."""
    from transformers.models.bert.modeling_bert import BertModel
    m = BertModel(bert_config(name, num_layers)).eval()
    for p in m.parameters():
        p.requires_grad_(False)
    return reinit_(m, seed)


def random_ids(batch, seq_len, vocab, seed=0):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (batch, seq_len), generator=g, dtype=torch.int64)


def varlen_lengths(batch=64, lo=8, hi=512, seed=0):
    """Per-sequence lengths uniform in [lo, hi] inclusive, from Python's random with the seed."""
    r = random.Random(seed)
    return [r.randint(lo, hi) for _ in range(batch)]


def varlen_ids(lengths, vocab, seed=0):
    g = torch.Generator().manual_seed(2000 + seed)
    return [torch.randint(0, vocab, (n,), generator=g, dtype=torch.int64) for n in lengths]


GPT2_CONFIGS = {
    # name: (layers, hidden, heads, vocab, positions)
    "gpt2-small": (12, 768, 12, 50257, 1024),
    "gpt2-tiny": (2, 128, 2, 1000, 128),
    "gpt2-mini": (2, 256, 4, 5003, 256),
}


def make_hf_gpt2(name="gpt2-small", seed=0, num_layers=None):
    """A HuggingFace GPT2Model (fp32, eval, CPU) with the seeded weights described at the top of this file."""
    from transformers.models.gpt2.modeling_gpt2 import GPT2Config, GPT2Model
    n, h, a, v, p = GPT2_CONFIGS[name]
    cfg = GPT2Config(vocab_size=v, n_positions=p, n_embd=h, n_layer=num_layers or n, n_head=a, resid_pdrop=0.0, embd_pdrop=0.0,
                     attn_pdrop=0.0, layer_norm_epsilon=1e-5, activation_function="gelu_new")
    m = GPT2Model(cfg).eval()
    for q in m.parameters():
        q.requires_grad_(False)
    return reinit_(m, seed)
