"""DistilBERT on the BERT kernels, with the class names and call signatures of the reference's
python/turbo_transformers/layers/modeling_distillbert.py (DistillBertAttention, DistrillFFN, DistrillTransformerBlock,
DistrillTransformer, DistilBertModel). Host composition only: attention = BertAttention with the block's sa_layer_norm,
feed-forward = the C++ DistrillFFN (positionwise_ffn.cpp:79-123). As in the reference the activation is the tanh-form GELU
and the embeddings stay the torch module; the 0/1 attention mask becomes the additive -10000 mask here.
"""
from typing import Optional, Sequence

import torch

from .._cxx import cxx
from .modeling_bert import BertAttention, _t
from .return_type import ReturnType, convert_returns_as_type
from .utils import AnyTensor, convert2tt_tensor, create_empty_if_none, try_convert, use_current_stream

__all__ = ['DistillBertAttention', 'DistrillFFN', 'DistrillTransformerBlock', 'DistrillTransformer', 'DistilBertModel']


class DistillBertAttention(BertAttention):
    def __call__(self, input_tensor: AnyTensor, attention_mask: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 output_attentions: Optional[bool] = False, return_type: Optional[ReturnType] = None,
                 is_trans_weight: Optional[bool] = False):
        if isinstance(attention_mask, torch.Tensor):  # [batch, keys] of 1 (attend) / 0 (padding)
            attention_mask = ((1.0 - attention_mask[:, None, None, :].float()) * -10000.0).contiguous()
        return super().__call__(input_tensor, attention_mask, head_mask, output_attentions, return_type, is_trans_weight)

    @staticmethod
    def from_torch(attention, layernorm: torch.nn.LayerNorm):
        p = {k: v.detach() for k, v in attention.named_parameters()}
        qkv_weight = torch.t(torch.cat((p['q_lin.weight'], p['k_lin.weight'], p['v_lin.weight']), 0)).contiguous().clone()
        qkv_bias = torch.cat((p['q_lin.bias'], p['k_lin.bias'], p['v_lin.bias']), 0).contiguous()
        return DistillBertAttention(convert2tt_tensor(qkv_weight), convert2tt_tensor(qkv_bias), convert2tt_tensor(_t(p['out_lin.weight'])),
                                    convert2tt_tensor(p['out_lin.bias']), convert2tt_tensor(layernorm.weight.detach()),
                                    convert2tt_tensor(layernorm.bias.detach()), attention.n_heads)


class DistrillFFN(cxx.DistrillFFN):
    def __call__(self, input_tensor: AnyTensor, return_type: Optional[ReturnType] = None, is_trans_weight: Optional[bool] = True,
                 output: Optional[cxx.Tensor] = None):
        input_tensor = try_convert(input_tensor)
        output = create_empty_if_none(output)
        super().__call__(input_tensor, output, is_trans_weight)
        return convert_returns_as_type(output, return_type)

    @staticmethod
    def from_torch(ffn, layernorm: torch.nn.LayerNorm, is_trans_weight: Optional[bool] = True):
        p = {k: v.detach() for k, v in ffn.named_parameters()}
        w1, w2 = (p['lin1.weight'], p['lin2.weight']) if is_trans_weight else (_t(p['lin1.weight']), _t(p['lin2.weight']))
        return DistrillFFN(convert2tt_tensor(w1.contiguous()), convert2tt_tensor(p['lin1.bias']), convert2tt_tensor(w2.contiguous()),
                           convert2tt_tensor(p['lin2.bias']), convert2tt_tensor(layernorm.weight.detach()),
                           convert2tt_tensor(layernorm.bias.detach()))


class DistrillTransformerBlock:
    def __init__(self, attn: DistillBertAttention, ffn: DistrillFFN):
        self.attention = attn
        self.ffn = ffn

    def __call__(self, hidden_states: AnyTensor, attention_mask: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 output_attentions=False, return_type: Optional[ReturnType] = None):
        attn_outputs = self.attention(hidden_states, attention_mask, head_mask, output_attentions=output_attentions,
                                      return_type=ReturnType.turbo_transformers)
        return (self.ffn(attn_outputs[0], return_type=return_type), ) + attn_outputs[1:]

    @staticmethod
    def from_torch(layer):
        return DistrillTransformerBlock(DistillBertAttention.from_torch(layer.attention, layer.sa_layer_norm),
                                        DistrillFFN.from_torch(layer.ffn, layer.output_layer_norm))


class DistrillTransformer:
    def __init__(self, blocks: Sequence[DistrillTransformerBlock]):
        self.blocks = blocks

    def __call__(self, hidden_states: AnyTensor, attention_mask: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 output_attentions: Optional[bool] = False, output_hidden_states: Optional[bool] = False,
                 return_type: Optional[ReturnType] = None):
        all_hidden_states, all_attentions = (), ()
        hidden_states = try_convert(hidden_states)
        for block in self.blocks:
            if output_hidden_states:
                all_hidden_states = all_hidden_states + (hidden_states, )
            out = block(hidden_states, attention_mask, None, output_attentions, ReturnType.turbo_transformers)
            hidden_states = out[0]
            if output_attentions:
                all_attentions = all_attentions + (out[1], )
        outputs = (convert_returns_as_type(hidden_states, return_type), )
        if output_hidden_states:
            outputs = outputs + (all_hidden_states, )
        if output_attentions:
            outputs = outputs + (all_attentions, )
        return outputs

    @staticmethod
    def from_torch(transform):
        return DistrillTransformer([DistrillTransformerBlock.from_torch(l) for l in transform.layer])


class DistilBertModel:
    def __init__(self, embeddings_onnxmodel_variant, inputmodel, backend="turbo"):
        if backend != "turbo":
            raise NotImplementedError("only the 'turbo' backend exists in this runtime")
        self.embeddings = embeddings_onnxmodel_variant  # the torch embeddings module, as in the reference
        self.turbo_transformer = inputmodel

    def __call__(self, input_ids: AnyTensor, attention_masks: Optional[AnyTensor] = None, token_type_ids: Optional[AnyTensor] = None,
                 position_ids: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 inputs_embeds: Optional[AnyTensor] = None, return_type: Optional[ReturnType] = None):
        use_current_stream(input_ids if isinstance(input_ids, torch.Tensor) else None)
        with torch.no_grad():
            hidden = self.embeddings(input_ids)
        return self.turbo_transformer(hidden_states=hidden.contiguous(), attention_mask=attention_masks, head_mask=head_mask,
                                      return_type=return_type)

    @staticmethod
    def from_torch(model, backend="turbo"):
        """`model`: a HuggingFace DistilBertModel already on the CUDA device and in the dtype to run in."""
        if backend != "turbo":
            raise NotImplementedError("only the 'turbo' backend exists in this runtime")
        if not next(model.parameters()).is_cuda:
            raise RuntimeError("the model must be on a CUDA device: this runtime has no CPU path")
        return DistilBertModel(model.embeddings, DistrillTransformer.from_torch(model.transformer), "turbo")
