"""Variable-length ("smart batch") BERT with the class names and call signatures of the reference's
python/turbo_transformers/layers/modeling_smart_pad.py. Tokens of all requests are packed as [1, sumL, H];
attention runs per sequence through a prefix-sum array instead of padded tensors, and the embedding runs
on the GPU in one pass (the reference embedded each sequence in torch and concatenated)."""
from typing import Optional, Sequence

import numpy as np
import torch

from .._cxx import cxx
from .modeling_bert import (BertEmbeddings, BertIntermediate, BertOutput, BertPooler, PoolingMap, PoolingType, _npz, _require_cuda,
                            _t, pack_qkv)
from .return_type import ReturnType, convert_returns_as_type
from .utils import AnyTensor, convert2tt_tensor, create_empty_if_none, try_convert, use_current_stream

__all__ = ['MultiHeadedAttentionSmartBatch', 'BertLayerSmartBatch', 'BertEncoderSmartBatch', 'BertModelSmartBatch',
           'BertModelNoPoolerSmartBatch']


def _empty():
    return cxx.Tensor.create_empty()


class MultiHeadedAttentionSmartBatch(cxx.MultiHeadedAttentionSmartBatch):
    def __call__(self, key_tensor: AnyTensor, value_tensor: AnyTensor, query_tensor: AnyTensor, query_seq_len_list: Sequence[int],
                 key_seq_len_list: Sequence[int], mask: Optional[AnyTensor] = None, layer_cache: Optional[dict] = None,
                 attn_type: str = None, pre_layernorm: bool = False, post_layernorm: bool = False, post_add_input: bool = False,
                 is_trans_weight: bool = False, return_type: Optional[ReturnType] = None, output: Optional[cxx.Tensor] = None,
                 attn: Optional[cxx.Tensor] = None, output_attentions: bool = False):
        """query_tensor is [1, sum(query_seq_len_list), hidden]. With mask=None keys beyond each sequence's
        length are excluded exactly (the reference built a [B,1,maxL] mask of -1e9 for the same effect)."""
        if isinstance(query_tensor, torch.Tensor):
            use_current_stream(query_tensor)
        key_tensor, value_tensor, query_tensor = try_convert(key_tensor), try_convert(value_tensor), try_convert(query_tensor)
        if mask is None and output_attentions and (attn_type or "self") == "self":
            lens = list(query_seq_len_list)
            m = torch.zeros(len(lens), 1, max(lens), dtype=torch.float32)
            for b, n in enumerate(lens):
                m[b, 0, n:] = -1e9
            mask = m.cuda()
        mask = try_convert(create_empty_if_none(mask))
        output, attn = create_empty_if_none(output), create_empty_if_none(attn)
        cache = {k: (try_convert(v) if v is not None else _empty()) for k, v in (layer_cache or {}).items()}
        attn_type = attn_type or "self"
        super().__call__(key_tensor, value_tensor, query_tensor, mask, attn_type, output,
                         attn if (output_attentions or attn_type == "context") else None, cache,
                         [int(n) for n in query_seq_len_list], [int(n) for n in key_seq_len_list], pre_layernorm, post_layernorm,
                         post_add_input, is_trans_weight)
        if layer_cache is not None and attn_type == "context":  # the projected encoder memory goes back to the caller's dict
            for k, v in cache.items():
                if "memory" in k and not v.is_null():
                    layer_cache[k] = convert_returns_as_type(v, ReturnType.TORCH)
        return convert_returns_as_type(output, return_type), attn

    @staticmethod
    def from_onmt(multi_headed_attn, layer_norm=None, is_trans_weight: bool = False):
        """From an OpenNMT-py style MultiHeadedAttention (linear_keys, linear_values, linear_query, final_linear, head_count),
        optionally with the block's LayerNorm (modeling_smart_pad.py:113-137 of the reference)."""
        from .modules import MultiHeadedAttention
        with torch.no_grad():
            packed = MultiHeadedAttention.pack_parameter(multi_headed_attn, is_trans_weight)
            if layer_norm is None:
                return MultiHeadedAttentionSmartBatch(*packed, multi_headed_attn.head_count)
            ln = {k: v.detach() for k, v in layer_norm.named_parameters()}
            return MultiHeadedAttentionSmartBatch(*packed, convert2tt_tensor(ln['weight']), convert2tt_tensor(ln['bias']),
                                                  multi_headed_attn.head_count)

    @staticmethod
    def from_torch(attention, layer_norm=None, is_trans_weight: bool = False):
        with torch.no_grad():
            qkv_weight, qkv_bias, p = pack_qkv(attention)
            g, b = p['output.LayerNorm.weight'], p['output.LayerNorm.bias']
            if layer_norm is not None:
                ln = {k: v.detach() for k, v in layer_norm.named_parameters()}
                g, b = ln['weight'], ln['bias']
            return MultiHeadedAttentionSmartBatch(_empty(), _empty(), _empty(), _empty(), _empty(), _empty(),
                                                  convert2tt_tensor(_t(p['output.dense.weight'])),
                                                  convert2tt_tensor(p['output.dense.bias']), convert2tt_tensor(qkv_weight),
                                                  convert2tt_tensor(qkv_bias), convert2tt_tensor(g), convert2tt_tensor(b),
                                                  attention.self.num_attention_heads)

    @staticmethod
    def from_npz(file_name: str, layer_num: int, num_attention_heads: int, device=None, dtype=None):
        f = np.load(file_name)
        pre = f'encoder.layer.{layer_num}.attention.'
        return MultiHeadedAttentionSmartBatch(_empty(), _empty(), _empty(), _empty(), _empty(), _empty(),
                                              _npz(f, pre + 'output.dense.weight', device, dtype),
                                              _npz(f, pre + 'output.dense.bias', device, dtype), _npz(f, pre + 'qkv.weight', device, dtype),
                                              _npz(f, pre + 'qkv.bias', device, dtype),
                                              _npz(f, pre + 'output.LayerNorm.weight', device, dtype),
                                              _npz(f, pre + 'output.LayerNorm.bias', device, dtype), num_attention_heads)


class BertLayerSmartBatch:
    def __init__(self, attention: MultiHeadedAttentionSmartBatch, intermediate: BertIntermediate, output: BertOutput):
        self.attention = attention
        self.intermediate = intermediate
        self.output = output

    def __call__(self, hidden_states: AnyTensor, query_seq_len_list: Sequence, attention_mask: Optional[AnyTensor] = None,
                 head_mask: Optional[AnyTensor] = None, output_attentions=False, return_type: Optional[ReturnType] = None):
        att_out, att_probs = self.attention(hidden_states, hidden_states, hidden_states, query_seq_len_list, [], mask=attention_mask,
                                            layer_cache=None, attn_type="self", post_layernorm=True,
                                            return_type=ReturnType.turbo_transformers, output_attentions=output_attentions)
        intermediate_output = self.intermediate(att_out, return_type=ReturnType.turbo_transformers)
        layer_output = self.output(intermediate_output, att_out, return_type=return_type)
        return (layer_output, att_probs) if output_attentions else (layer_output, )

    @staticmethod
    def from_torch(layer):
        return BertLayerSmartBatch(MultiHeadedAttentionSmartBatch.from_torch(layer.attention),
                                   BertIntermediate.from_torch(layer.intermediate), BertOutput.from_torch(layer.output))

    @staticmethod
    def from_npz(file_name: str, layer_num: int, num_attention_heads: int, device=None, dtype=None):
        return BertLayerSmartBatch(MultiHeadedAttentionSmartBatch.from_npz(file_name, layer_num, num_attention_heads, device, dtype),
                                   BertIntermediate.from_npz(file_name, layer_num, device, dtype),
                                   BertOutput.from_npz(file_name, layer_num, device, dtype))


class BertEncoderSmartBatch:
    def __init__(self, layer: Sequence[BertLayerSmartBatch]):
        self.layer = layer

    def __call__(self, hidden_states: AnyTensor, query_seq_len_list: Sequence, attention_mask: Optional[AnyTensor] = None,
                 head_mask: Optional[AnyTensor] = None, output_attentions: Optional[bool] = False,
                 output_hidden_states: Optional[bool] = False, return_type: Optional[ReturnType] = None):
        all_hidden_states, all_attentions = (), ()
        hidden_states = try_convert(hidden_states)
        attention_mask = try_convert(attention_mask)
        lens = [int(n) for n in query_seq_len_list]
        for l in self.layer:
            layer_outputs = l(hidden_states=hidden_states, query_seq_len_list=lens, attention_mask=attention_mask,
                              output_attentions=output_attentions, return_type=ReturnType.turbo_transformers)
            if output_hidden_states:
                all_hidden_states = all_hidden_states + (hidden_states, )
            hidden_states = layer_outputs[0]
            if output_attentions:
                all_attentions = all_attentions + (layer_outputs[1], )
        outputs = (convert_returns_as_type(hidden_states, return_type), )
        if output_hidden_states:
            outputs = outputs + (all_hidden_states, )
        if output_attentions:
            outputs = outputs + (all_attentions, )
        return outputs

    @staticmethod
    def from_torch(encoder):
        return BertEncoderSmartBatch([BertLayerSmartBatch.from_torch(l) for l in encoder.layer])

    @staticmethod
    def from_npz(file_name: str, num_hidden_layers: int, num_attention_heads: int, device=None, dtype=None):
        return BertEncoderSmartBatch([BertLayerSmartBatch.from_npz(file_name, i, num_attention_heads, device, dtype)
                                      for i in range(num_hidden_layers)])


def pack_ids(inputs, device=None):
    """A list of [1, L_i] / [L_i] id tensors (or one already-packed 1-D tensor) -> int64 [sumL] on the GPU."""
    if isinstance(inputs, torch.Tensor):
        ids = inputs.reshape(-1)
    else:
        ids = torch.cat([torch.as_tensor(i).reshape(-1) for i in inputs])
    if not ids.is_cuda:
        ids = ids.to(device if device is not None else "cuda", non_blocking=True)
    return ids.to(torch.int64).contiguous()


class BertModelNoPoolerSmartBatch:
    def __init__(self, embeddings: BertEmbeddings, encoder: BertEncoderSmartBatch):
        self.embeddings = embeddings
        self.encoder = encoder

    def __call__(self, inputs: Sequence[torch.Tensor], query_seq_len_list: Sequence, attention_masks: Optional[AnyTensor] = None,
                 token_type_ids: Optional[AnyTensor] = None, position_ids: Optional[AnyTensor] = None,
                 head_mask: Optional[AnyTensor] = None, inputs_embeds: Optional[AnyTensor] = None,
                 output_attentions: Optional[bool] = None, output_hidden_states: Optional[bool] = None,
                 pooling_type: PoolingType = PoolingType.FIRST, return_type: Optional[ReturnType] = None):
        """inputs: one id tensor per request (or a packed 1-D tensor); positions restart at 0 per request."""
        lens = [int(n) for n in query_seq_len_list]
        assert len(lens) != 0
        ids = pack_ids(inputs)
        use_current_stream(ids)
        hidden = cxx.Tensor.create_empty()
        # segment and position ids are packed the same way as the ids (one per token, requests back to back)
        pos = convert2tt_tensor(pack_ids(position_ids)) if position_ids is not None else cxx.Tensor.create_empty()
        types = convert2tt_tensor(pack_ids(token_type_ids)) if token_type_ids is not None else cxx.Tensor.create_empty()
        self.embeddings.packed(convert2tt_tensor(ids), lens, hidden, pos, types)
        return self.encoder(hidden_states=hidden, query_seq_len_list=lens, attention_mask=attention_masks,
                            output_attentions=output_attentions, output_hidden_states=output_hidden_states, return_type=return_type)

    @staticmethod
    def from_torch(model, device: Optional[torch.device] = None):
        _require_cuda(model, device)
        return BertModelNoPoolerSmartBatch(BertEmbeddings.from_torch(model.embeddings), BertEncoderSmartBatch.from_torch(model.encoder))

    @staticmethod
    def from_npz(file_name: str, config, device: Optional[torch.device] = None, dtype=None):
        return BertModelNoPoolerSmartBatch(BertEmbeddings.from_npz(file_name, device, dtype),
                                           BertEncoderSmartBatch.from_npz(file_name, config.num_hidden_layers,
                                                                          config.num_attention_heads, device, dtype))


class BertModelSmartBatch:
    def __init__(self, model: BertModelNoPoolerSmartBatch, pooler: BertPooler, config=None):
        self.config = config
        self.bertmodel_nopooler = model
        self.pooler = pooler

    def __call__(self, inputs: AnyTensor, query_seq_len_list: Sequence, attention_masks: Optional[AnyTensor] = None,
                 token_type_ids: Optional[AnyTensor] = None, position_ids: Optional[AnyTensor] = None,
                 head_mask: Optional[AnyTensor] = None, inputs_embeds: Optional[AnyTensor] = None,
                 output_attentions: Optional[bool] = None, output_hidden_states: Optional[bool] = None,
                 pooling_type: PoolingType = PoolingType.FIRST, pooler_output: Optional[AnyTensor] = None,
                 return_type: Optional[ReturnType] = None):
        """Returns (sequence_output [1, sumL, H], pooler_output [B, H], ...). The pooled row of request b is
        taken from ITS first (last/mean/max) token; the reference pooled the packed tensor as if it were one
        sequence, which yields only request 0's row -- row 0 here is identical to that."""
        lens = [int(n) for n in query_seq_len_list]
        encoder_outputs = self.bertmodel_nopooler(inputs, lens, attention_masks, token_type_ids, position_ids,
                                                  inputs_embeds=inputs_embeds, output_attentions=output_attentions,
                                                  output_hidden_states=output_hidden_states, pooling_type=pooling_type,
                                                  return_type=ReturnType.turbo_transformers)
        sequence_output = encoder_outputs[0]
        pooled_in = cxx.Tensor.create_empty()
        cxx.SequencePool(PoolingMap[pooling_type]).packed(sequence_output, lens, pooled_in)
        pooler_output = self.pooler(pooled_in, return_type, pooler_output)
        return (convert_returns_as_type(sequence_output, return_type), pooler_output) + encoder_outputs[1:]

    @staticmethod
    def from_torch(model, device: Optional[torch.device] = None):
        _require_cuda(model, device)
        nopooler = BertModelNoPoolerSmartBatch(BertEmbeddings.from_torch(model.embeddings),
                                               BertEncoderSmartBatch.from_torch(model.encoder))
        return BertModelSmartBatch(nopooler, BertPooler.from_torch(model.pooler), model.config)

    @staticmethod
    def from_pretrained(model_id_or_path: str, device: Optional[torch.device] = None):
        from transformers.models.bert.modeling_bert import BertModel as TorchBertModel
        torch_model = TorchBertModel.from_pretrained(model_id_or_path)
        model = BertModelSmartBatch.from_torch(torch_model, device)
        model._torch_model = torch_model
        return model

    @staticmethod
    def from_npz(file_name: str, config, device=None, dtype=None):
        return BertModelSmartBatch(BertModelNoPoolerSmartBatch.from_npz(file_name, config, device, dtype),
                                   BertPooler.from_npz(file_name, device, dtype), config)
