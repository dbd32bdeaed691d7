"""int8 BERT ("qbert") with the class names of the reference's python/turbo_transformers/layers/qmodeling_bert.py.

The reference quantised only the two feed-forward Linears, through torch's CPU dynamic quantisation, and
re-applied the bias with native epilogues (qmodeling_bert.py:13-45). Here every Linear can run as an int8
tensor-core GEMM: per-tensor symmetric weights (scale = max|W|/127), per-row dynamic symmetric activations,
int32 accumulation, and an epilogue that dequantises, adds the bias and applies GELU or the residual in
fp16/bf16. Attention scores, softmax and layer norms stay in 16-bit/fp32.
`quantize_attention=False` restricts int8 to the feed-forward Linears, as the reference did.
"""
from typing import Optional

import torch

from .modeling_bert import (BertAttention, BertEmbeddings, BertEncoder, BertIntermediate, BertLayer, BertModel, BertModelNoPooler,
                            BertOutput, BertPooler, _require_cuda)

__all__ = ['QBertIntermediate', 'QBertOutput', 'QBertLayer', 'QBertEncoder', 'QBertModel']


class QBertIntermediate(BertIntermediate):
    @staticmethod
    def from_torch(intermediate):
        base = BertIntermediate.from_torch(intermediate)
        base.quantize_int8()
        base.__class__ = QBertIntermediate
        return base


class QBertOutput(BertOutput):
    @staticmethod
    def from_torch(output):
        base = BertOutput.from_torch(output)
        base.quantize_int8()
        base.__class__ = QBertOutput
        return base


class QBertLayer(BertLayer):
    @staticmethod
    def from_torch(layer, quantize_attention: bool = True):
        attention = BertAttention.from_torch(layer.attention)
        if quantize_attention:
            attention.quantize_int8()
        return QBertLayer(attention, QBertIntermediate.from_torch(layer.intermediate), QBertOutput.from_torch(layer.output))


class QBertEncoder(BertEncoder):
    @staticmethod
    def from_torch(encoder, quantize_attention: bool = True):
        return QBertEncoder([QBertLayer.from_torch(l, quantize_attention) for l in encoder.layer])


class QBertModel(BertModel):
    @staticmethod
    def from_torch(model, device: Optional[torch.device] = None, backend: Optional[str] = None,
                   quantize_attention: bool = True):
        """model: a HuggingFace BertModel in fp16 or bf16 (the dtype of the non-GEMM math and of the outputs)."""
        if backend not in (None, "turbo"):
            raise NotImplementedError("only the 'turbo' backend exists in this runtime")
        _require_cuda(model, device)
        if next(model.parameters()).dtype == torch.float32:
            raise RuntimeError("the int8 path dequantises to fp16/bf16: convert the model with .half() or .bfloat16() first")
        nopooler = BertModelNoPooler(BertEmbeddings.from_torch(model.embeddings),
                                     QBertEncoder.from_torch(model.encoder, quantize_attention))
        return QBertModel(nopooler, BertPooler.from_torch(model.pooler), "turbo", model.config)
