"""RoBERTa on the BERT kernels: torch embeddings (RoBERTa's padding-offset position ids) + BertEncoder + BertPooler, as in
the reference's python/turbo_transformers/layers/modeling_roberta.py:52-149. Unlike the reference, which hands the encoder
an empty mask whatever the caller passed, a caller-supplied attention mask is applied.
"""
from typing import Optional

import torch

from .modeling_bert import BertEncoder, BertPooler, PoolingMap, PoolingType, SequencePool
from .return_type import ReturnType, convert_returns_as_type
from .utils import AnyTensor, use_current_stream

__all__ = ['RobertaModel']


class RobertaModel:
    def __init__(self, embeddings, encoder: BertEncoder, pooler: BertPooler, config):
        self.config = config
        self.embeddings = embeddings
        self.encoder = encoder
        self.pooler = pooler

    def __call__(self, input_ids: AnyTensor, attention_mask: Optional[torch.Tensor] = None, token_type_ids: Optional[torch.Tensor] = None,
                 position_ids: Optional[torch.Tensor] = None, head_mask: Optional[torch.Tensor] = None,
                 inputs_embeds: Optional[torch.Tensor] = None, pooling_type: PoolingType = PoolingType.FIRST,
                 hidden_cache: Optional[AnyTensor] = None, output: Optional[AnyTensor] = None, return_type: Optional[ReturnType] = None):
        if input_ids is not None and inputs_embeds is not None:
            raise ValueError("You cannot specify both input_ids and inputs_embeds at the same time")
        if input_ids is None and inputs_embeds is None:
            raise ValueError("You have to specify either input_ids or inputs_embeds")
        assert head_mask is None
        use_current_stream(input_ids if input_ids is not None else inputs_embeds)
        with torch.no_grad():
            hidden = self.embeddings(input_ids=input_ids, position_ids=position_ids, token_type_ids=token_type_ids,
                                     inputs_embeds=inputs_embeds)
        ext_mask = None
        if attention_mask is not None:
            ext_mask = ((1.0 - attention_mask[:, None, None, :].float()) * -10000.0).contiguous()
        encoder_outputs = self.encoder(hidden_states=hidden.contiguous(), attention_mask=ext_mask, return_type=ReturnType.turbo_transformers)
        sequence_output = encoder_outputs[0]
        pooled = SequencePool(PoolingMap[pooling_type])(input_tensor=sequence_output, return_type=ReturnType.turbo_transformers)
        pooler_output = self.pooler(pooled, return_type)
        return (convert_returns_as_type(sequence_output, return_type), pooler_output) + encoder_outputs[1:]

    @staticmethod
    def from_torch(model, device: Optional[torch.device] = None):
        """`model`: a HuggingFace RobertaModel (with pooler); it is moved to `device` when one is given."""
        if device is not None:
            model.to(device)
        if not next(model.parameters()).is_cuda:
            raise RuntimeError("the model must be on a CUDA device: this runtime has no CPU path")
        return RobertaModel(model.embeddings, BertEncoder.from_torch(model.encoder), BertPooler.from_torch(model.pooler), model.config)
