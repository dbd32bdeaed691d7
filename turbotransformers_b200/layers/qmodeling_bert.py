"""int8 BERT ("qbert") with the class names of the reference's python/turbo_transformers/layers/qmodeling_bert.py.

Two schemes:

  scheme="reference"  The reference's own recipe (qmodeling_bert.py:13-45): only the two feed-forward Linears are
      quantised, with torch's dynamic quantisation arithmetic restated on the GPU -- per-tensor symmetric qint8 weights
      (scale = max|W| / 127.5), per-tensor affine activations over the whole [tokens, K] tensor with 7-bit levels (the
      x86 engines' reduce_range) and a zero point, int32 accumulation, then bias + GELU / bias + residual + LayerNorm.
      Attention stays in the model's floating dtype, as the reference keeps it in fp32.
  scheme="benchmark"  (default) Every Linear runs as an int8 tensor-core GEMM: per-tensor symmetric weights
      (scale = max|W| / 127), per-row dynamic symmetric activations, int32 accumulation, and an epilogue that dequantises,
      adds the bias and applies GELU or the residual. `quantize_attention=False` restricts it to the feed-forward Linears.

Attention scores, softmax and layer norms stay in 16-bit/fp32 in both.
"""
from typing import Optional

import torch

from .modeling_bert import (BertAttention, BertEmbeddings, BertEncoder, BertIntermediate, BertLayer, BertModel, BertModelNoPooler,
                            BertOutput, BertPooler, _require_cuda)

__all__ = ['QBertIntermediate', 'QBertOutput', 'QBertLayer', 'QBertEncoder', 'QBertModel']

_MODES = {"benchmark": 1, "reference": 2}


def _mode(scheme):
    if scheme not in _MODES:
        raise ValueError(f"unknown int8 scheme {scheme!r}: expected one of {sorted(_MODES)}")
    return _MODES[scheme]


class QBertIntermediate(BertIntermediate):
    @staticmethod
    def from_torch(intermediate, scheme: str = "benchmark"):
        base = BertIntermediate.from_torch(intermediate)
        base.quantize_int8(_mode(scheme))
        base.__class__ = QBertIntermediate
        return base


class QBertOutput(BertOutput):
    @staticmethod
    def from_torch(output, scheme: str = "benchmark"):
        base = BertOutput.from_torch(output)
        base.quantize_int8(_mode(scheme))
        base.__class__ = QBertOutput
        return base


class QBertLayer(BertLayer):
    @staticmethod
    def from_torch(layer, quantize_attention: bool = True, scheme: str = "benchmark"):
        attention = BertAttention.from_torch(layer.attention)
        if quantize_attention and scheme == "benchmark":
            attention.quantize_int8()
        return QBertLayer(attention, QBertIntermediate.from_torch(layer.intermediate, scheme), QBertOutput.from_torch(layer.output, scheme))


class QBertEncoder(BertEncoder):
    @staticmethod
    def from_torch(encoder, quantize_attention: bool = True, scheme: str = "benchmark"):
        return QBertEncoder([QBertLayer.from_torch(l, quantize_attention, scheme) for l in encoder.layer])


class QBertModel(BertModel):
    @staticmethod
    def from_torch(model, device: Optional[torch.device] = None, backend: Optional[str] = None,
                   quantize_attention: bool = True, scheme: str = "benchmark"):
        """model: a HuggingFace BertModel in fp16 or bf16 (the dtype of the non-GEMM math and of the outputs).
        scheme: "benchmark" or "reference" (see the module docstring); "reference" never quantises attention."""
        if backend not in (None, "turbo"):
            raise NotImplementedError("only the 'turbo' backend exists in this runtime")
        _mode(scheme)
        _require_cuda(model, device)
        if next(model.parameters()).dtype == torch.float32:
            raise RuntimeError("the int8 path dequantises to fp16/bf16: convert the model with .half() or .bfloat16() first")
        nopooler = BertModelNoPooler(BertEmbeddings.from_torch(model.embeddings),
                                     QBertEncoder.from_torch(model.encoder, quantize_attention, scheme))
        return QBertModel(nopooler, BertPooler.from_torch(model.pooler), "turbo", model.config)
