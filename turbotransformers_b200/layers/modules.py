"""MultiHeadedAttention and PositionwiseFeedForward with the call signatures of the reference's
python/turbo_transformers/layers/modules.py:36-243: self attention (with the in-place "self_keys"/"self_values" decoding
cache for 16-bit models) and context (encoder-decoder) attention with its "memory_keys"/"memory_values" cache."""
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
        attn_type = attn_type or "self"
        super().__call__(key_tensor, value_tensor, query_tensor, mask, attn_type, output,
                         attn if (output_attentions or attn_type == "context") else None, cache, pre_layernorm,
                         post_layernorm, post_add_input, is_trans_weight)
        if layer_cache is not None:
            # the caches go back to the caller's dict, as the reference does (modules.py:79-83): the projected encoder memory
            # as torch tensors [B, heads, Lk, d]; the self-attention cache as the runtime's own tensor (its buffer is paged and
            # reserved ahead, so it is handed back as it is and passed in again on the next step)
            for k, v in cache.items():
                if v.is_null():
                    continue
                if "memory" in k and attn_type == "context":
                    layer_cache[k] = convert_returns_as_type(v, ReturnType.TORCH)
                elif "self" in k and attn_type == "self":
                    layer_cache[k] = v
        return convert_returns_as_type(output, return_type), attn

    @staticmethod
    def pack_parameter(multi_headed_attn, is_trans_weight: Optional[bool] = False):
        """The ten weight tensors of an OpenNMT-py style attention module (parameters linear_keys / linear_values /
        linear_query / final_linear), in the constructor's order (modules.py:90-141 of the reference)."""
        p = {k: v.detach() for k, v in multi_headed_attn.named_parameters()}
        if getattr(multi_headed_attn, "max_relative_positions", 0) != 0:
            raise ValueError("multi_headed_attn's max_relative_positions should be 0!")
        w = (lambda t: t.contiguous()) if is_trans_weight else (lambda t: torch.t(t).contiguous())
        qkv_weight = w(torch.cat((p['linear_query.weight'], p['linear_keys.weight'], p['linear_values.weight']), 0))
        qkv_bias = torch.cat((p['linear_query.bias'], p['linear_keys.bias'], p['linear_values.bias']), 0).contiguous()
        T = convert2tt_tensor
        return (T(w(p['linear_keys.weight'])), T(p['linear_keys.bias']), T(w(p['linear_values.weight'])), T(p['linear_values.bias']),
                T(w(p['linear_query.weight'])), T(p['linear_query.bias']), T(w(p['final_linear.weight'])), T(p['final_linear.bias']),
                T(qkv_weight), T(qkv_bias))

    @staticmethod
    def from_onmt(multi_headed_attn, layer_norm=None, is_trans_weight: bool = False):
        """From an OpenNMT-py style MultiHeadedAttention (any module with linear_keys, linear_values, linear_query,
        final_linear and head_count), optionally with the block's LayerNorm (modules.py:143-167 of the reference)."""
        with torch.no_grad():
            packed = MultiHeadedAttention.pack_parameter(multi_headed_attn, is_trans_weight)
            if layer_norm is None:
                return MultiHeadedAttention(*packed, multi_headed_attn.head_count)
            ln = {k: v.detach() for k, v in layer_norm.named_parameters()}
            return MultiHeadedAttention(*packed, convert2tt_tensor(ln['weight']), convert2tt_tensor(ln['bias']),
                                        multi_headed_attn.head_count)

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

    @staticmethod
    def from_onmt(position_wise_ffn, is_trans_weight: Optional[bool] = True):
        """From an OpenNMT-py style PositionwiseFeedForward (parameters w_1, w_2, layer_norm; modules.py:277-309 of the
        reference). With is_trans_weight the torch [out, in] matrices are used as they are: call with the same flag."""
        p = {k: v.detach() for k, v in position_wise_ffn.named_parameters()}
        w = (lambda t: t.contiguous()) if is_trans_weight else (lambda t: torch.t(t).contiguous())
        T = convert2tt_tensor
        with torch.no_grad():
            return PositionwiseFeedForward(T(w(p['w_1.weight'])), T(p['w_1.bias']), T(w(p['w_2.weight'])), T(p['w_2.bias']),
                                           T(p['layer_norm.weight']), T(p['layer_norm.bias']))
