"""TEST INFRASTRUCTURE ONLY -- drives the compiled, unmodified reference CPU code (oracle/_ref).

The reference's Python package cannot be imported on this image (it imports `onmt`, which is absent),
so this file talks to the reference's pybind module directly and repeats the weight packing its
`from_torch` constructors do (python/turbo_transformers/layers/modeling_bert.py:58-65,88-95,124-131,
179-204,530-560; modeling_smart_pad.py:434-486).  Nothing in the product package may import this file.
"""
import importlib.util
import os
import sys

import numpy as np
import torch
import torch.utils.dlpack as dlpack

HERE = os.path.dirname(os.path.abspath(__file__))
_cxx = None
_device = "cpu"   # where T() puts tensors; "cuda" only after use_cuda_build()


def available():
    from . import build_ref
    return os.path.exists(build_ref.module_path())


def cuda_build_available():
    from . import build_ref
    return os.path.exists(build_ref.cuda_module_path())


def use_cuda_build():
    """Make this process drive the reference's GPU build (oracle/_ref/cuda) with tensors on cuda:0.

    The CPU and GPU builds export the same C++ types, so a process can hold only one of them: call this before
    anything else here has loaded the CPU build.
    """
    global _device
    if _cxx is not None and _device != "cuda":
        raise RuntimeError("the reference's CPU build is already loaded in this process")
    _device = "cuda"
    return load()


def load():
    """Import oracle/_ref/turbo_transformers_cxx (building it first if the reference tree is present)."""
    global _cxx
    if _cxx is not None:
        return _cxx
    from . import build_ref
    if _device == "cuda":
        path = build_ref.build_cuda(verbose=False)
    else:
        path = build_ref.build(verbose=False)
    if path is None or not os.path.exists(path):
        raise RuntimeError("oracle/_ref is not built and the reference tree is not available")
    # The OpenBLAS object was linked against a libgfortran that sits beside it but is not on the loader
    # path: load those dependencies first.
    import ctypes
    import glob
    blas = build_ref.find_openblas()
    if blas:
        for pat in ("libquadmath*", "libgfortran*"):
            for dep in sorted(glob.glob(os.path.join(os.path.dirname(blas), pat))):
                try:
                    ctypes.CDLL(dep, mode=ctypes.RTLD_GLOBAL)
                except OSError:
                    pass
    spec = importlib.util.spec_from_file_location("turbo_transformers_cxx", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _cxx = mod
    return mod


def set_num_threads(n):
    load().set_num_threads(int(n))


def T(t):
    """torch tensor (or numpy array) -> reference core::Tensor owning a private copy on the driver's device."""
    if isinstance(t, np.ndarray):
        t = torch.from_numpy(np.ascontiguousarray(t))
    t = t.detach().contiguous()
    t = t.clone() if t.device.type == _device else t.to(_device)
    return load().Tensor.from_dlpack(dlpack.to_dlpack(t))


def back(t):
    return dlpack.from_dlpack(t.to_dlpack())


def E():
    return load().Tensor.create_empty()


def pack_bert_weights(hf_model):
    """HF BertModel -> the dict-of-numpy layout both oracles use (weights [in,out], fused QKV [H,3H])."""
    def n(p):
        return p.detach().float().cpu().numpy().copy()
    e = hf_model.embeddings
    W = {"embedding": {"word": n(e.word_embeddings.weight), "position": n(e.position_embeddings.weight),
                       "token_type": n(e.token_type_embeddings.weight), "ln_gamma": n(e.LayerNorm.weight),
                       "ln_beta": n(e.LayerNorm.bias)}, "layers": []}
    for l in hf_model.encoder.layer:
        a = l.attention
        qkv_w = torch.t(torch.cat((a.self.query.weight, a.self.key.weight, a.self.value.weight), 0)).contiguous()
        qkv_b = torch.cat((a.self.query.bias, a.self.key.bias, a.self.value.bias), 0)
        W["layers"].append({
            "attention": {"qkv_weight": n(qkv_w), "qkv_bias": n(qkv_b),
                          "dense_weight": n(torch.t(a.output.dense.weight).contiguous()),
                          "dense_bias": n(a.output.dense.bias), "ln_gamma": n(a.output.LayerNorm.weight),
                          "ln_beta": n(a.output.LayerNorm.bias)},
            "inter_weight": n(torch.t(l.intermediate.dense.weight).contiguous()),
            "inter_bias": n(l.intermediate.dense.bias),
            "out_weight": n(torch.t(l.output.dense.weight).contiguous()), "out_bias": n(l.output.dense.bias),
            "out_ln_gamma": n(l.output.LayerNorm.weight), "out_ln_beta": n(l.output.LayerNorm.bias)})
    if getattr(hf_model, "pooler", None) is not None:
        W["pooler_weight"] = n(torch.t(hf_model.pooler.dense.weight).contiguous())
        W["pooler_bias"] = n(hf_model.pooler.dense.bias)
    return W


class RefBert:
    """The reference's BERT, fixed-length and smart-batch, assembled from its compiled layer classes."""

    def __init__(self, W, num_heads):
        cxx = load()
        self.cxx, self.h = cxx, num_heads
        e = W["embedding"]
        self.emb = cxx.BERTEmbedding(T(e["word"]), T(e["position"]), T(e["token_type"]), T(e["ln_gamma"]),
                                     T(e["ln_beta"]))
        self.layers, self.sb_layers = [], []
        for lw in W["layers"]:
            a = lw["attention"]
            att = cxx.BertAttention(T(a["qkv_weight"]), T(a["qkv_bias"]), T(a["dense_weight"]), T(a["dense_bias"]),
                                    T(a["ln_gamma"]), T(a["ln_beta"]), num_heads)
            H = a["dense_weight"].shape[0]
            qw, kw, vw = (np.ascontiguousarray(a["qkv_weight"][:, i * H:(i + 1) * H]) for i in range(3))
            qb, kb, vb = (np.ascontiguousarray(a["qkv_bias"][i * H:(i + 1) * H]) for i in range(3))
            sb = cxx.MultiHeadedAttentionSmartBatch(T(kw), T(kb), T(vw), T(vb), T(qw), T(qb), T(a["dense_weight"]),
                                                    T(a["dense_bias"]), T(a["qkv_weight"]), T(a["qkv_bias"]),
                                                    T(a["ln_gamma"]), T(a["ln_beta"]), num_heads)
            inter = cxx.BertIntermediate(T(lw["inter_weight"]), T(lw["inter_bias"]))
            out = cxx.BertOutput(T(lw["out_weight"]), T(lw["out_bias"]), T(lw["out_ln_gamma"]),
                                 T(lw["out_ln_beta"]))
            self.layers.append((att, inter, out))
            self.sb_layers.append((sb, inter, out))
        self.pooler = cxx.BertPooler(T(W["pooler_weight"]), T(W["pooler_bias"])) if "pooler_weight" in W else None
        self.prep, self.seqpool = cxx.PrepareBertMasks(), cxx.SequencePool("First")

    def embed(self, ids, att_mask=None):
        am = T(att_mask) if att_mask is not None else E()
        tt, pos, ext = E(), E(), E()
        x = T(ids)
        self.prep(x, am, tt, pos, ext)
        h = E()
        self.emb(x, pos, tt, h)
        return h, ext

    def forward(self, ids, att_mask=None, n_layers=None):
        """ids int64 [B,L] -> (sequence_output [B,L,H], pooled [B,H]) as torch fp32."""
        h, ext = self.embed(torch.as_tensor(ids, dtype=torch.int64), att_mask)
        for att, inter, out in self.layers[:n_layers]:
            ao, ap, io, ho = E(), E(), E(), E()
            att(h, ext, ao, ap, False)
            inter(ao, io)
            out(io, ao, ho)
            h = ho
        pooled = None
        if self.pooler is not None:
            sp, po = E(), E()
            self.seqpool(h, sp)
            self.pooler(sp, po)
            pooled = back(po)
        return back(h), pooled

    def forward_smart_batch(self, id_list, n_layers=None):
        """list of int64 id sequences -> packed [1,sumL,H] (modeling_smart_pad.py:434-486)."""
        lens = [int(len(i)) for i in id_list]
        xs = []
        for ids in id_list:
            h, _ = self.embed(torch.as_tensor(ids, dtype=torch.int64).reshape(1, -1))
            xs.append(back(h))
        x = torch.cat(xs, 1)
        mask = torch.zeros(len(lens), 1, max(lens))
        for b, n in enumerate(lens):
            mask[b, 0, n:] = -1e9
        return self.smart_batch_layers(x, mask, lens, n_layers)

    def smart_batch_layers(self, x, mask, lens, n_layers=None):
        """The encoder stack over an already embedded, packed batch x [1,sumL,H] with its additive mask [B,1,maxL]."""
        h, m = T(x), T(mask)
        for sb, inter, out in self.sb_layers[:n_layers]:
            ao, ap, io, ho = E(), E(), E(), E()
            sb(h, h, h, m, "self", ao, ap, {}, lens, [], False, True, False, False)
            inter(ao, io)
            out(io, ao, ho)
            h = ho
        return back(h)


class RefQBertRecipe:
    """The reference's int8 recipe, layer by layer (python/turbo_transformers/layers/qmodeling_bert.py:13-45,158-192):
    torch dynamic quantisation of the two feed-forward Linears with the bias stripped, the bias re-applied by the compiled
    reference's FusedAddBiasGELU / FusedAddBiasLayerNorm, attention through its fp32 BertAttention."""

    def __init__(self, hf_model):
        import warnings
        cxx = load()
        W = pack_bert_weights(hf_model)
        self.ref = RefBert(W, hf_model.config.num_attention_heads)
        self.layers = []
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            for l in hf_model.encoder.layer:
                qi = torch.quantization.quantize_dynamic(l.intermediate, {torch.nn.Linear}, dtype=torch.qint8)
                qo = torch.quantization.quantize_dynamic(l.output, {torch.nn.Linear}, dtype=torch.qint8)
                wi, _ = qi.dense._weight_bias()
                qi.dense.set_weight_bias(wi, None)
                wo, _ = qo.dense._weight_bias()
                qo.dense.set_weight_bias(wo, None)
                gelu = cxx.FusedAddBiasGELU(T(l.intermediate.dense.bias))
                lnorm = cxx.FusedAddBiasLayerNorm(T(l.output.dense.bias), T(l.output.LayerNorm.weight), T(l.output.LayerNorm.bias))
                self.layers.append((qi.dense, qo.dense, gelu, lnorm))

    def embed(self, ids):
        """int64 ids [B, L] -> (embedding output as torch fp32 [B, L, H], the additive mask tensor for layer())."""
        h, ext = self.ref.embed(torch.as_tensor(ids, dtype=torch.int64))
        return back(h).clone(), ext

    def layer(self, i, h, ext):
        """One encoder layer of the recipe on the torch fp32 hidden states h."""
        att = self.ref.layers[i][0]
        qi, qo, gelu, lnorm = self.layers[i]
        ao, ap = E(), E()
        att(T(h), ext, ao, ap, False)
        a = back(ao).clone()
        inter = T(qi(a))
        gelu(inter)
        out = T(qo(back(inter).clone()))
        lnorm(T(a), out)
        return back(out).clone()

    def forward(self, ids):
        h, ext = self.embed(ids)
        for i in range(len(self.layers)):
            h = self.layer(i, h, ext)
        return h


def context_attention_weights(hidden, seed=0):
    """Seeded fp32 weights of one attention layer in the layout restate.context_attention takes ([in,out] matrices)."""
    r = np.random.default_rng(seed)
    w = {}
    for n in ("q", "k", "v"):
        w[n + "_weight"] = (r.standard_normal((hidden, hidden)) * 0.05).astype(np.float32)
        w[n + "_bias"] = (r.standard_normal(hidden) * 0.02).astype(np.float32)
    w["dense_weight"] = (r.standard_normal((hidden, hidden)) * 0.05).astype(np.float32)
    w["dense_bias"] = (r.standard_normal(hidden) * 0.02).astype(np.float32)
    w["ln_gamma"] = (1.0 + 0.1 * r.standard_normal(hidden)).astype(np.float32)
    w["ln_beta"] = (0.1 * r.standard_normal(hidden)).astype(np.float32)
    return w


class RefContextAttention:
    """The reference's MultiHeadedAttention driven with attn_type="context" (multi_headed_attention.cpp:45-167,260-380)."""

    def __init__(self, w, num_heads):
        cxx = load()
        qkv_w = np.ascontiguousarray(np.concatenate([w["q_weight"], w["k_weight"], w["v_weight"]], 1))
        qkv_b = np.concatenate([w["q_bias"], w["k_bias"], w["v_bias"]])
        self.att = cxx.MultiHeadedAttention(T(w["k_weight"]), T(w["k_bias"]), T(w["v_weight"]), T(w["v_bias"]), T(w["q_weight"]),
                                            T(w["q_bias"]), T(w["dense_weight"]), T(w["dense_bias"]), T(qkv_w), T(qkv_b),
                                            T(w["ln_gamma"]), T(w["ln_beta"]), num_heads)

    def __call__(self, query, key, value, mask, memory=None, keep_memory=False, pre_layernorm=False, post_layernorm=False,
                 post_add_input=False):
        """-> (output, att_score, (memory_keys, memory_values) or None) as numpy. memory = a pair a previous call returned."""
        out, score = E(), E()
        cache = {}
        if memory is not None:
            cache = {"memory_keys": T(memory[0]), "memory_values": T(memory[1])}
        elif keep_memory:
            cache = {"memory_keys": E(), "memory_values": E()}
        self.att(T(key), T(value), T(query), T(mask) if mask is not None else E(), "context", out, score, cache, pre_layernorm,
                 post_layernorm, post_add_input, False)
        mem = (back(cache["memory_keys"]).cpu().numpy().copy(), back(cache["memory_values"]).cpu().numpy().copy()) if cache else None
        return back(out).cpu().numpy().copy(), back(score).cpu().numpy().copy(), mem


def decoder_layer_weights(hidden, ffn_dim, seed=0):
    """Seeded fp32 weights of one decoder layer in the layout restate.transformer_decoder_layer takes."""
    r = np.random.default_rng(seed + 100)
    ctx = context_attention_weights(hidden, seed)
    sw = context_attention_weights(hidden, seed + 1)
    self_w = {"qkv_weight": np.ascontiguousarray(np.concatenate([sw["q_weight"], sw["k_weight"], sw["v_weight"]], 1)),
              "qkv_bias": np.concatenate([sw["q_bias"], sw["k_bias"], sw["v_bias"]]), "dense_weight": sw["dense_weight"],
              "dense_bias": sw["dense_bias"], "ln_gamma": sw["ln_gamma"], "ln_beta": sw["ln_beta"], "split": sw}
    ffn = {"w1_weight": (r.standard_normal((hidden, ffn_dim)) * 0.05).astype(np.float32),
           "w1_bias": (r.standard_normal(ffn_dim) * 0.02).astype(np.float32),
           "w2_weight": (r.standard_normal((ffn_dim, hidden)) * 0.05).astype(np.float32),
           "w2_bias": (r.standard_normal(hidden) * 0.02).astype(np.float32),
           "ln_gamma": (1.0 + 0.1 * r.standard_normal(hidden)).astype(np.float32),
           "ln_beta": (0.1 * r.standard_normal(hidden)).astype(np.float32)}
    return {"self": self_w, "context": ctx, "ffn": ffn}


class RefDecoderLayer:
    """The reference's layer classes composed as python/turbo_transformers/layers/modeling_decoder.py:58-140 composes them."""

    def __init__(self, lw, num_heads):
        cxx = load()
        sw = lw["self"]["split"]
        self.self_attn = cxx.MultiHeadedAttention(T(sw["k_weight"]), T(sw["k_bias"]), T(sw["v_weight"]), T(sw["v_bias"]), T(sw["q_weight"]),
                                                  T(sw["q_bias"]), T(sw["dense_weight"]), T(sw["dense_bias"]), T(lw["self"]["qkv_weight"]),
                                                  T(lw["self"]["qkv_bias"]), T(sw["ln_gamma"]), T(sw["ln_beta"]), num_heads)
        self.context = RefContextAttention(lw["context"], num_heads)
        f = lw["ffn"]
        self.ffn = cxx.PositionwiseFeedForward(T(f["w1_weight"]), T(f["w1_bias"]), T(f["w2_weight"]), T(f["w2_bias"]), T(f["ln_gamma"]),
                                               T(f["ln_beta"]))

    def __call__(self, x, memory_bank, src_mask, dec_mask):
        query, score = E(), E()
        xt = T(x)
        self.self_attn(xt, xt, xt, T(dec_mask) if dec_mask is not None else E(), "self", query, score, {}, True, False, True, False)
        mid, attn, _ = self.context(back(query).numpy(), memory_bank, memory_bank, src_mask, pre_layernorm=True, post_add_input=True)
        out = E()
        self.ffn(T(mid), out, False)
        return back(out).numpy().copy(), attn[:, 0]


def pack_gpt2_weights(hf_model):
    """HF GPT2Model -> the dict layout oracle/restate.py:gpt2_model takes (Conv1D weights are already [in,out])."""
    def n(p):
        return p.detach().float().cpu().numpy().copy()
    W = {"wte": n(hf_model.wte.weight), "wpe": n(hf_model.wpe.weight), "lnf_gamma": n(hf_model.ln_f.weight),
         "lnf_beta": n(hf_model.ln_f.bias), "layers": []}
    for b in hf_model.h:
        W["layers"].append({
            "attention": {"qkv_weight": n(b.attn.c_attn.weight), "qkv_bias": n(b.attn.c_attn.bias),
                          "dense_weight": n(b.attn.c_proj.weight), "dense_bias": n(b.attn.c_proj.bias),
                          "ln_gamma": n(b.ln_1.weight), "ln_beta": n(b.ln_1.bias)},
            "ln2_gamma": n(b.ln_2.weight), "ln2_beta": n(b.ln_2.bias), "fc_weight": n(b.mlp.c_fc.weight),
            "fc_bias": n(b.mlp.c_fc.bias), "proj_weight": n(b.mlp.c_proj.weight), "proj_bias": n(b.mlp.c_proj.bias)})
    return W
