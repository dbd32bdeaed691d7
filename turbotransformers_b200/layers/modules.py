"""MultiHeadedAttention and PositionwiseFeedForward with the call signatures of the reference's
python/turbo_transformers/layers/modules.py:36-243. Only self attention is in scope; the NMT decoder's
context attention and incremental caches raise."""
from typing import Optional

import torch

from .._cxx import cxx
from .modeling_bert import _t, pack_qkv
from .return_type import ReturnType, convert_returns_as_type
from .utils import AnyTensor, convert2tt_tensor, create_empty_if_none, try_convert, use_current_stream

__all__ = ['MultiHeadedAttention', 'PositionwiseFeedForward']


def _empty():
    return cxx.Tensor.create_empty()


class MultiHeadedAttention(cxx.MultiHeadedAttention):
    def __call__(self, key_tensor: AnyTensor, value_tensor: AnyTensor, query_tensor: AnyTensor, mask: Optional[AnyTensor] = None,
                 layer_cache: Optional[dict] = None, attn_type: str = None, pre_layernorm: bool = False,
                 post_layernorm: bool = False, post_add_input: bool = False, is_trans_weight: bool = False,
                 return_type: Optional[ReturnType] = None, output: Optional[cxx.Tensor] = None, attn: Optional[cxx.Tensor] = None,
                 output_attentions: bool = False):
        """Returns (output, attn). `attn` holds the attention probabilities only for fp32 models or when
        output_attentions is set; otherwise it is a null tensor (the fused kernel never writes them)."""
        if isinstance(query_tensor, torch.Tensor):
            use_current_stream(query_tensor)
        key_tensor, value_tensor, query_tensor = try_convert(key_tensor), try_convert(value_tensor), try_convert(query_tensor)
        mask = try_convert(create_empty_if_none(mask))
        output, attn = create_empty_if_none(output), create_empty_if_none(attn)
        cache = {k: (try_convert(v) if v is not None else _empty()) for k, v in (layer_cache or {}).items()}
        self.set_materialize_scores(bool(output_attentions))
        super().__call__(key_tensor, value_tensor, query_tensor, mask, attn_type or "self", output, attn, cache, pre_layernorm,
                         post_layernorm, post_add_input, is_trans_weight)
        return convert_returns_as_type(output, return_type), attn

    @staticmethod
    def from_torch(attention, layer_norm=None, is_trans_weight: bool = False):
        """From a HuggingFace BertAttention. `layer_norm` (a torch LayerNorm) replaces the attention's own
        output LayerNorm when given, e.g. a pre-LN block's first norm."""
        with torch.no_grad():
            qkv_weight, qkv_bias, p = pack_qkv(attention)
            out_w = _t(p['output.dense.weight'])
            if is_trans_weight:
                qkv_weight = torch.cat((p['self.query.weight'], p['self.key.weight'], p['self.value.weight']), 0).contiguous()
                out_w = p['output.dense.weight'].contiguous()
            if layer_norm is not None:
                ln = {k: v.detach() for k, v in layer_norm.named_parameters()}
                g, b = ln['weight'], ln['bias']
            else:
                g, b = p['output.LayerNorm.weight'], p['output.LayerNorm.bias']
            return MultiHeadedAttention(_empty(), _empty(), _empty(), _empty(), _empty(), _empty(), convert2tt_tensor(out_w),
                                        convert2tt_tensor(p['output.dense.bias']), convert2tt_tensor(qkv_weight),
                                        convert2tt_tensor(qkv_bias), convert2tt_tensor(g), convert2tt_tensor(b),
                                        attention.self.num_attention_heads)


class PositionwiseFeedForward(cxx.PositionwiseFeedForward):
    def __call__(self, input_tensor: AnyTensor, return_type: Optional[ReturnType] = None, is_trans_weight: Optional[bool] = True,
                 output: Optional[cxx.Tensor] = None):
        input_tensor = try_convert(input_tensor)
        output = create_empty_if_none(output)
        super().__call__(input_tensor, output, is_trans_weight)
        return convert_returns_as_type(output, return_type)
