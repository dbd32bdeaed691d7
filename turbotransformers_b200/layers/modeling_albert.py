"""ALBERT on the BERT kernels, with the class names of the reference's python/turbo_transformers/layers/modeling_albert.py
(AlbertAttention, AlbertLayer, AlbertLayerGroup, AlbertTransformer, AlbertModel). Host composition only: attention =
BertAttention (fused QKV, output projection, residual LayerNorm), the rest of a layer = the C++ AlbertLayer
(albert_layer.cpp:31-50). As in the reference, the embeddings, the embedding-to-hidden projection and the pooler Linear stay
torch modules; layers are shared through the layer groups exactly as the torch model shares them.
"""
from typing import Optional, Sequence

import torch

from .._cxx import cxx
from .modeling_bert import BertAttention, _t
from .return_type import ReturnType, convert_returns_as_type
from .utils import AnyTensor, convert2tt_tensor, create_empty_if_none, try_convert, use_current_stream

__all__ = ['AlbertAttention', 'AlbertLayer', 'AlbertLayerGroup', 'AlbertTransformer', 'AlbertModel']


class AlbertAttention(BertAttention):
    @staticmethod
    def from_torch(attention):
        p = {k: v.detach() for k, v in attention.named_parameters()}
        qkv_weight = torch.t(torch.cat((p['query.weight'], p['key.weight'], p['value.weight']), 0)).contiguous().clone()
        qkv_bias = torch.cat((p['query.bias'], p['key.bias'], p['value.bias']), 0).contiguous()
        return AlbertAttention(convert2tt_tensor(qkv_weight), convert2tt_tensor(qkv_bias), convert2tt_tensor(_t(p['dense.weight'])),
                               convert2tt_tensor(p['dense.bias']), convert2tt_tensor(p['LayerNorm.weight']),
                               convert2tt_tensor(p['LayerNorm.bias']), attention.num_attention_heads)


class AlbertLayer(cxx.AlbertLayer):
    def __init__(self, attention: AlbertAttention, ffn, ffn_bias, ffn_output, ffn_ouput_bias, fl, fl_bias):
        self.attention = attention
        super().__init__(ffn, ffn_bias, ffn_output, ffn_ouput_bias, fl, fl_bias)

    def __call__(self, input_tensor: AnyTensor, attention_mask: AnyTensor, head_mask: AnyTensor = None,
                 output_attentions: Optional[bool] = False, output_hidden_states: Optional[bool] = False,
                 return_type: Optional[ReturnType] = ReturnType.TORCH, attention_output: Optional[AnyTensor] = None):
        if head_mask is not None:
            raise ValueError("head mask must be None")
        att = self.attention(input_tensor, attention_mask, output_attentions=output_attentions, return_type=ReturnType.turbo_transformers)
        hidden_output, hidden_states = cxx.Tensor.create_empty(), cxx.Tensor.create_empty()
        super().__call__(att[0], hidden_output, hidden_states)
        out = (convert_returns_as_type(hidden_states, return_type), )
        return out + (att[1], ) if output_attentions else out

    @staticmethod
    def from_torch(layer):
        return AlbertLayer(AlbertAttention.from_torch(layer.attention), convert2tt_tensor(_t(layer.ffn.weight)),
                           convert2tt_tensor(layer.ffn.bias.detach()), convert2tt_tensor(_t(layer.ffn_output.weight)),
                           convert2tt_tensor(layer.ffn_output.bias.detach()), convert2tt_tensor(layer.full_layer_layer_norm.weight.detach()),
                           convert2tt_tensor(layer.full_layer_layer_norm.bias.detach()))


class AlbertLayerGroup:
    def __init__(self, layers: Sequence[AlbertLayer]):
        self.albert_layers = layers

    def __call__(self, hidden_states: AnyTensor, attention_mask: AnyTensor, head_mask: AnyTensor = None, output_attentions: bool = False,
                 output_hidden_states: bool = False, return_type: Optional[ReturnType] = ReturnType.TORCH):
        layer_attentions = ()
        hidden_states = try_convert(hidden_states)
        for layer in self.albert_layers:
            out = layer(hidden_states, attention_mask, None, output_attentions, output_hidden_states, ReturnType.turbo_transformers)
            hidden_states = out[0]
            if output_attentions:
                layer_attentions = layer_attentions + (out[1], )
        outputs = (convert_returns_as_type(hidden_states, return_type), )
        return outputs + (layer_attentions, ) if output_attentions else outputs

    @staticmethod
    def from_torch(group):
        return AlbertLayerGroup([AlbertLayer.from_torch(l) for l in group.albert_layers])


class AlbertTransformer:
    def __init__(self, embedding_hidden_mapping_in: torch.nn.Linear, albert_layer_groups: Sequence[AlbertLayerGroup], config):
        self.config = config
        self.embedding_hidden_mapping_in = embedding_hidden_mapping_in
        self.albert_layer_groups = albert_layer_groups

    def __call__(self, hidden_states: AnyTensor, attention_mask: AnyTensor, head_mask: AnyTensor = None, output_attentions: bool = False,
                 output_hidden_states: bool = False, return_type: Optional[ReturnType] = ReturnType.TORCH):
        with torch.no_grad():
            hidden_states = try_convert(self.embedding_hidden_mapping_in(hidden_states).contiguous())
        attention_mask = try_convert(create_empty_if_none(attention_mask))
        all_attentions = ()
        per_group = self.config.num_hidden_layers // self.config.num_hidden_groups
        for i in range(self.config.num_hidden_layers):
            out = self.albert_layer_groups[i // per_group](hidden_states, attention_mask, None, output_attentions, output_hidden_states,
                                                           ReturnType.turbo_transformers)
            hidden_states = out[0]
            if output_attentions:
                all_attentions = all_attentions + out[-1]
        outputs = (convert_returns_as_type(hidden_states, return_type), )
        return outputs + (all_attentions, ) if output_attentions else outputs

    @staticmethod
    def from_torch(encoder):
        return AlbertTransformer(encoder.embedding_hidden_mapping_in, [AlbertLayerGroup.from_torch(g) for g in encoder.albert_layer_groups],
                                 encoder.config)


class AlbertModel:
    def __init__(self, embeddings, encoder: AlbertTransformer, pooler: torch.nn.Linear, config):
        self.config = config
        self.embeddings = embeddings
        self.encoder = encoder
        self.pooler = pooler

    def __call__(self, input_ids: AnyTensor, attention_mask: Optional[torch.Tensor] = None, token_type_ids: Optional[torch.Tensor] = None,
                 position_ids: Optional[torch.Tensor] = None, head_mask: Optional[torch.Tensor] = None,
                 inputs_embeds: Optional[torch.Tensor] = None, return_type: Optional[ReturnType] = ReturnType.TORCH):
        assert head_mask is None
        use_current_stream(input_ids if input_ids is not None else inputs_embeds)
        ext_mask = None
        if attention_mask is not None:
            ext_mask = ((1.0 - attention_mask[:, None, None, :].float()) * -10000.0).contiguous()
        with torch.no_grad():
            emb = self.embeddings(input_ids, position_ids=position_ids, token_type_ids=token_type_ids, inputs_embeds=inputs_embeds)
        sequence_output = self.encoder(emb, ext_mask, return_type=ReturnType.TORCH)[0]
        with torch.no_grad():
            pooled = torch.tanh(self.pooler(sequence_output[:, 0]))
        return (sequence_output, pooled)

    @staticmethod
    def from_torch(model):
        """`model`: a HuggingFace AlbertModel already on the CUDA device and in the dtype to run in."""
        if not next(model.parameters()).is_cuda:
            raise RuntimeError("the model must be on a CUDA device: this runtime has no CPU path")
        return AlbertModel(model.embeddings, AlbertTransformer.from_torch(model.encoder), model.pooler, model.config)
