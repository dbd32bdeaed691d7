"""Regenerates the golden vectors in this directory by running the compiled, unmodified reference CPU code
(oracle/_ref, built by oracle/build_ref.py from the reference tree) on seeded synthetic models.

    python tests/golden/make_golden.py

Each .npz holds the seeds/config needed to rebuild the model and inputs (see
turbotransformers_b200/synthetic.py) and the reference's outputs in fp32. Nothing else is stored: weights
are regenerated from the seed on any machine.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import ref_driver  # noqa: E402
from turbotransformers_b200 import synthetic  # noqa: E402

torch.set_grad_enabled(False)


def save(name, **kw):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **kw)
    print(f"{name}: {os.path.getsize(path) / 1024:.0f} KiB")


def bert_fixed(name, model_name, seed, batch, seq_len, mask_tail=0):
    hf = synthetic.make_hf_bert(model_name, seed)
    W = ref_driver.pack_bert_weights(hf)
    ids = synthetic.random_ids(batch, seq_len, hf.config.vocab_size, seed)
    ref = ref_driver.RefBert(W, hf.config.num_attention_heads)
    att_mask = None
    if mask_tail:
        att_mask = torch.ones(batch, seq_len, dtype=torch.int64)
        for b in range(batch):
            att_mask[b, seq_len - (b % (mask_tail + 1)):] = 0
    seq, pooled = ref.forward(ids, att_mask)
    save(name, model=model_name, seed=seed, ids=ids.numpy(), att_mask=(att_mask.numpy() if att_mask is not None else np.zeros(0)),
         sequence_output=seq.numpy(), pooled_output=pooled.numpy())


def bert_smart(name, model_name, seed, lens):
    hf = synthetic.make_hf_bert(model_name, seed)
    W = ref_driver.pack_bert_weights(hf)
    ids = synthetic.varlen_ids(lens, hf.config.vocab_size, seed)
    ref = ref_driver.RefBert(W, hf.config.num_attention_heads)
    out = ref.forward_smart_batch(ids)
    save(name, model=model_name, seed=seed, lens=np.array(lens), ids=torch.cat(ids).numpy(), sequence_output=out.numpy()[0])


def bert_layers(name, model_name, seed, batch, seq_len):
    """Per-layer-class outputs (embedding, attention incl. probabilities, intermediate, output) of layer 0."""
    hf = synthetic.make_hf_bert(model_name, seed, num_layers=1)
    W = ref_driver.pack_bert_weights(hf)
    ids = synthetic.random_ids(batch, seq_len, hf.config.vocab_size, seed)
    ref = ref_driver.RefBert(W, hf.config.num_attention_heads)
    E, back = ref_driver.E, ref_driver.back
    att_mask = torch.ones(batch, seq_len, dtype=torch.int64)
    att_mask[-1, seq_len - 3:] = 0
    h, ext = ref.embed(ids, att_mask)
    att, inter, out = ref.layers[0]
    ao, ap, io, ho = E(), E(), E(), E()
    att(h, ext, ao, ap, False)
    inter(ao, io)
    out(io, ao, ho)
    emb_np = back(h).numpy()
    save(name, model=model_name, seed=seed, ids=ids.numpy(), att_mask=att_mask.numpy(), embedding=emb_np,
         attention_output=back(ao).numpy().copy(), attention_probs=back(ap).numpy(), intermediate=back(io).numpy(),
         layer_output=back(ho).numpy())


def qbert_reference_recipe(name, model_name, seed, batch, seq_len):
    """The reference's own int8 recipe (python/turbo_transformers/layers/qmodeling_bert.py:13-45,158-192):
    torch dynamic quantisation of the two feed-forward Linears with the bias stripped, the bias re-applied by
    the reference's native FusedAddBiasGELU / FusedAddBiasLayerNorm, fp32 attention."""
    hf = synthetic.make_hf_bert(model_name, seed)
    ids = synthetic.random_ids(batch, seq_len, hf.config.vocab_size, seed)
    h = ref_driver.RefQBertRecipe(hf).forward(ids)
    save(name, model=model_name, seed=seed, ids=ids.numpy(), sequence_output=h.numpy())


if __name__ == "__main__":
    ref_driver.set_num_threads(8)
    bert_fixed("bert_base_b1_s128", "bert-base", 0, 1, 128)                 # benchmark config 1
    bert_fixed("bert_mini_b3_s50_masked", "bert-mini", 1, 3, 50, mask_tail=7)
    bert_smart("bert_base_smart_37_5_64", "bert-base", 0, [37, 5, 64])      # packed variable length
    bert_smart("bert_mini_smart_4_1", "bert-mini", 2, [4, 1])               # lens of bert_smart_batch_test.py
    bert_smart("bert_mini_smart_9_7_13", "bert-mini", 3, [9, 7, 13])        # lens of multi_head_attn_smart_batch_test.py
    bert_layers("bert_mini_layer0_b2_s16", "bert-mini", 4, 2, 16)
    qbert_reference_recipe("qbert_recipe_bert_base_b1_s128", "bert-base", 0, 1, 128)
