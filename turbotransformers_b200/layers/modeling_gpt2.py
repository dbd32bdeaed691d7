"""GPT-2 decoder stack built from the same layer classes: full-sequence forward, and incremental decoding over a
key/value cache (`past`), the decoder's `layer_cache` path of the reference's MultiHeadedAttention.

The reference's GPT2Model wraps onnxruntime only and raises for its own "turbo" backend
(python/turbo_transformers/layers/modeling_gpt2.py:39-40,57-58). This class composes the block the way the
reference composes pre-LN blocks for its NMT encoder (modeling_encoder.py:81-91): MultiHeadedAttention with
pre_layernorm + post_add_input and a causal mask, then a pre-LN feed-forward with the tanh-form GELU
(equal to GPT-2's gelu_new), a final LayerNorm, and logits = hidden . wte^T (MatMul with b_trans).
"""
from typing import Optional

import torch

from .._cxx import cxx
from .return_type import ReturnType, convert_returns_as_type
from .utils import AnyTensor, convert2tt_tensor, try_convert, use_current_stream

__all__ = ['GPT2Model']


def _empty():
    return cxx.Tensor.create_empty()


class GPT2Model:
    def __init__(self, embedding, blocks, final_norm, lm_head, config, backend="turbo"):
        if backend != "turbo":
            raise NotImplementedError("only the 'turbo' backend exists in this runtime")
        self.embedding, self.blocks, self.final_norm, self.lm_head, self.config = embedding, blocks, final_norm, lm_head, config
        self.backend = backend
        self.dtype = config.torch_dtype_of_weights

    def new_cache(self):
        """An empty key/value cache for incremental decoding (16-bit models): one `layer_cache` dict per block. Pass it as `past`
        with the prompt first, then with each new token (or few tokens); it grows in place."""
        if self.dtype == torch.float32:
            raise NotImplementedError("incremental decoding is provided for fp16 / bf16 models")
        return [{"self_keys": _empty(), "self_values": _empty()} for _ in self.blocks]

    @staticmethod
    def cached_length(past) -> int:
        k = past[0]["self_keys"]
        return 0 if k.is_null() else k.shape(0)

    def __call__(self, input_ids: AnyTensor, return_logits: bool = True, return_type: Optional[ReturnType] = None, past=None,
                 contiguous_logits: bool = True):
        """input_ids int64 [B, L] on the GPU -> (last_hidden_state [B,L,H], logits [B,L,vocab] or None).
        With `past` (from new_cache()), input_ids are the tokens that follow what the cache already holds.
        contiguous_logits=False returns the logits as a view of rows padded to a multiple of 8 entries (torch tensors only):
        a 50257-entry row does not start on a 16-byte boundary, and making the rows contiguous costs a second pass over
        the largest tensor of the model."""
        if isinstance(input_ids, torch.Tensor):
            use_current_stream(input_ids)
        ids = try_convert(input_ids)
        x = _empty()
        self.embedding(ids, x, self.cached_length(past) if past is not None else 0)
        mask = _empty()
        if past is not None and self.dtype == torch.float32:
            raise NotImplementedError("incremental decoding is provided for fp16 / bf16 models")
        if self.dtype == torch.float32:
            # the exact-precision path applies an explicit additive mask, as the reference's kernels do
            B, L = ids.shape(0), ids.shape(1)
            m = torch.triu(torch.full((L, L), -10000.0, dtype=torch.float32, device="cuda"), 1)
            mask = convert2tt_tensor(m.unsqueeze(0).repeat(B, 1, 1).contiguous())
        for i, (attn, ffn) in enumerate(self.blocks):
            a, y = _empty(), _empty()
            # no score tensor is asked for (None): 16-bit models run the fused attention kernel; pre-LN, + input
            attn(x, x, x, mask, "self", a, None, past[i] if past is not None else {}, True, False, True, False)
            ffn(a, y, False)
            x = y
        h = _empty()
        self.final_norm(x, h)
        logits = None
        if return_logits and not contiguous_logits and return_type in (None, ReturnType.TORCH):
            padded = _empty()
            self.lm_head.padded(h, padded)
            logits = convert_returns_as_type(padded, ReturnType.TORCH)[..., :self.lm_head.width()]
        elif return_logits:
            logits = _empty()
            self.lm_head(h, logits)
            logits = convert_returns_as_type(logits, return_type)
        return convert_returns_as_type(h, return_type), logits

    @staticmethod
    def from_torch(model, device: Optional[torch.device] = None, backend: Optional[str] = None):
        """model: a HuggingFace GPT2Model (or the .transformer of a GPT2LMHeadModel) on a CUDA device.
        HuggingFace stores GPT-2 projections as Conv1D weights [in, out], the layout these layers take."""
        if backend not in (None, "turbo"):
            raise NotImplementedError("only the 'turbo' backend exists in this runtime")
        if device is None:
            device = next(model.parameters()).device
        if torch.device(device).type != 'cuda':
            raise RuntimeError("this runtime computes on CUDA devices only (no CPU path)")
        model.to(device)
        cfg = model.config
        cfg.torch_dtype_of_weights = model.wte.weight.dtype
        eps = float(cfg.layer_norm_epsilon)
        T = lambda p: convert2tt_tensor(p.detach().contiguous())
        blocks = []
        for blk in model.h:
            attn = cxx.MultiHeadedAttention(_empty(), _empty(), _empty(), _empty(), _empty(), _empty(), T(blk.attn.c_proj.weight),
                                            T(blk.attn.c_proj.bias), T(blk.attn.c_attn.weight), T(blk.attn.c_attn.bias),
                                            T(blk.ln_1.weight), T(blk.ln_1.bias), cfg.n_head)
            attn.set_pre_layernorm_eps(eps)
            attn.set_causal(True)
            ffn = cxx.PositionwiseFeedForward(T(blk.mlp.c_fc.weight), T(blk.mlp.c_fc.bias), T(blk.mlp.c_proj.weight),
                                              T(blk.mlp.c_proj.bias), T(blk.ln_2.weight), T(blk.ln_2.bias))
            ffn.set_activation("gelu")
            ffn.set_layernorm_eps(eps)
            blocks.append((attn, ffn))
        embedding = cxx.TokenPositionEmbedding(T(model.wte.weight), T(model.wpe.weight))
        final_norm = cxx.LayerNorm(T(model.ln_f.weight), T(model.ln_f.bias), eps)
        lm_head = cxx.Linear(T(model.wte.weight), _empty(), True)  # tied embedding, stored [vocab, hidden]
        return GPT2Model(embedding, blocks, final_norm, lm_head, cfg)
