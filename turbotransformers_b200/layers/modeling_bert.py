"""BERT layers and model with the class names, call signatures and `from_torch` / `from_npz` loaders of
the reference's python/turbo_transformers/layers/modeling_bert.py. The compute is in the C++ layer classes
(csrc/host/layers.h); this file only re-packs HuggingFace weights and hands tensors over through DLPack.

Weight layout kept from the reference: Linear weights are stored [in, out]; the attention q, k, v
projections are fused into one [hidden, 3*hidden] matrix with column blocks q|k|v and a [3*hidden] bias.
The dtype of the torch model (fp32, fp16 or bf16) selects the kernel family.
"""
import enum
from typing import Optional, Sequence

import numpy as np
import torch

from .._cxx import cxx
from .return_type import ReturnType, convert_returns_as_type
from .utils import (AnyTensor, convert2tt_tensor, create_empty_if_none, to_param_dict, to_param_dict_convert_tt, try_convert,
                    use_current_stream)

__all__ = ['BertEmbeddings', 'BertIntermediate', 'BertOutput', 'BertAttention', 'BertLayer', 'BertEncoder', 'SequencePool',
           'BertModel', 'BertModelNoPooler', 'PoolingType', 'PoolingMap', 'BertPooler']


def _t(w: torch.Tensor) -> torch.Tensor:
    """[out, in] torch Linear weight -> contiguous [in, out] copy."""
    return torch.t(w.detach()).contiguous().clone()


def _npz(f, key, device, dtype=None):
    a = torch.from_numpy(np.ascontiguousarray(f[key]))
    if dtype is not None and a.is_floating_point():
        a = a.to(dtype)
    return convert2tt_tensor(a.to(device if device is not None else "cuda").contiguous())


class BertEmbeddings(cxx.BERTEmbedding):
    def __call__(self, input_ids: AnyTensor, position_ids: AnyTensor, token_type_ids: AnyTensor,
                 return_type: Optional[ReturnType] = None, output: Optional[cxx.Tensor] = None):
        input_ids = try_convert(input_ids)
        position_ids = try_convert(create_empty_if_none(position_ids))
        token_type_ids = try_convert(create_empty_if_none(token_type_ids))
        output = create_empty_if_none(output)
        super().__call__(input_ids, position_ids, token_type_ids, output)
        return convert_returns_as_type(output, return_type)

    @staticmethod
    def from_torch(bert_embedding) -> 'BertEmbeddings':
        params = to_param_dict_convert_tt(bert_embedding)
        return BertEmbeddings(params['word_embeddings.weight'], params['position_embeddings.weight'],
                              params['token_type_embeddings.weight'], params['LayerNorm.weight'], params['LayerNorm.bias'])

    @staticmethod
    def from_npz(file_name: str, device: Optional[torch.device] = None, dtype=None):
        f = np.load(file_name)
        return BertEmbeddings(*(_npz(f, 'embeddings.' + k, device, dtype) for k in
                                ('word_embeddings.weight', 'position_embeddings.weight', 'token_type_embeddings.weight',
                                 'LayerNorm.weight', 'LayerNorm.bias')))


class BertIntermediate(cxx.BertIntermediate):
    def __call__(self, input_tensor: AnyTensor, return_type: Optional[ReturnType] = None, output: Optional[cxx.Tensor] = None):
        input_tensor = try_convert(input_tensor)
        output = create_empty_if_none(output)
        super().__call__(input_tensor, output)
        return convert_returns_as_type(output, return_type)

    @staticmethod
    def from_torch(intermediate):
        p = to_param_dict(intermediate)
        return BertIntermediate(convert2tt_tensor(_t(p["dense.weight"])), convert2tt_tensor(p['dense.bias']))

    @staticmethod
    def from_npz(file_name: str, layer_num: int, device: Optional[torch.device] = None, dtype=None):
        f = np.load(file_name)
        pre = f'encoder.layer.{layer_num}.intermediate.dense.'
        return BertIntermediate(_npz(f, pre + 'weight', device, dtype), _npz(f, pre + 'bias', device, dtype))


class BertOutput(cxx.BertOutput):
    def __call__(self, intermediate_output: AnyTensor, attention_output: AnyTensor, return_type: Optional[ReturnType] = None,
                 output: Optional[cxx.Tensor] = None):
        intermediate_output = try_convert(intermediate_output)
        attention_output = try_convert(attention_output)
        output = create_empty_if_none(output)
        super().__call__(intermediate_output, attention_output, output)
        return convert_returns_as_type(output, return_type)

    @staticmethod
    def from_torch(output):
        p = to_param_dict(output)
        return BertOutput(convert2tt_tensor(_t(p["dense.weight"])), convert2tt_tensor(p["dense.bias"]),
                          convert2tt_tensor(p["LayerNorm.weight"]), convert2tt_tensor(p["LayerNorm.bias"]))

    @staticmethod
    def from_npz(file_name: str, layer_num: int, device: Optional[torch.device] = None, dtype=None):
        f = np.load(file_name)
        pre = f'encoder.layer.{layer_num}.output.'
        return BertOutput(*(_npz(f, pre + k, device, dtype) for k in
                            ('dense.weight', 'dense.bias', 'LayerNorm.weight', 'LayerNorm.bias')))


def pack_qkv(attention):
    """(qkv_weight [H,3H], qkv_bias [3H]) from a HuggingFace BertAttention, q|k|v column blocks."""
    p = {k: v.detach() for k, v in attention.named_parameters()}
    qkv_weight = torch.t(torch.cat((p['self.query.weight'], p['self.key.weight'], p['self.value.weight']), 0)).contiguous().clone()
    qkv_bias = torch.cat((p['self.query.bias'], p['self.key.bias'], p['self.value.bias']), 0).contiguous()
    return qkv_weight, qkv_bias, p


class BertAttention(cxx.BertAttention):
    def __call__(self, input_tensor: AnyTensor, attention_mask: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 output_attentions: Optional[bool] = False, return_type: Optional[ReturnType] = None,
                 is_trans_weight: Optional[bool] = False):
        """Self attention + output projection + residual layer norm. Returns (context_layer[, attention_probs]).
        attention_probs are produced only when output_attentions is set (16-bit models then take the
        unfused path, which materialises them)."""
        assert head_mask is None
        input_tensor = try_convert(input_tensor)
        attention_mask = try_convert(create_empty_if_none(attention_mask))
        context_layer = cxx.Tensor.create_empty()
        attn_probs = cxx.Tensor.create_empty()
        super().__call__(input_tensor, attention_mask, context_layer, attn_probs if output_attentions else None, is_trans_weight)
        if output_attentions:
            return (convert_returns_as_type(context_layer, return_type),
                    convert_returns_as_type(attn_probs, ReturnType.turbo_transformers))
        return (convert_returns_as_type(context_layer, return_type), )

    @staticmethod
    def from_torch(attention):
        with torch.no_grad():
            qkv_weight, qkv_bias, p = pack_qkv(attention)
            return BertAttention(convert2tt_tensor(qkv_weight), convert2tt_tensor(qkv_bias),
                                 convert2tt_tensor(_t(p['output.dense.weight'])), convert2tt_tensor(p['output.dense.bias']),
                                 convert2tt_tensor(p['output.LayerNorm.weight']), convert2tt_tensor(p['output.LayerNorm.bias']),
                                 attention.self.num_attention_heads)

    @staticmethod
    def from_npz(file_name: str, layer_num: int, num_attention_heads: int, device: Optional[torch.device] = None, dtype=None):
        f = np.load(file_name)
        pre = f'encoder.layer.{layer_num}.attention.'
        return BertAttention(*(_npz(f, pre + k, device, dtype) for k in
                               ('qkv.weight', 'qkv.bias', 'output.dense.weight', 'output.dense.bias', 'output.LayerNorm.weight',
                                'output.LayerNorm.bias')), num_attention_heads)


class BertLayer:
    def __init__(self, attention: BertAttention, intermediate: BertIntermediate, output: BertOutput):
        self.attention = attention
        self.intermediate = intermediate
        self.output = output

    def __call__(self, hidden_states: AnyTensor, attention_mask: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 output_attentions=False, return_type: Optional[ReturnType] = None):
        self_attention_outputs = self.attention(hidden_states, attention_mask, head_mask, output_attentions=output_attentions,
                                                return_type=ReturnType.turbo_transformers)
        attention_output = self_attention_outputs[0]
        intermediate_output = self.intermediate(attention_output, return_type=ReturnType.turbo_transformers)
        layer_output = self.output(intermediate_output, attention_output, return_type=return_type)
        return (layer_output, ) + self_attention_outputs[1:]

    @staticmethod
    def from_torch(layer):
        return BertLayer(BertAttention.from_torch(layer.attention), BertIntermediate.from_torch(layer.intermediate),
                         BertOutput.from_torch(layer.output))

    @staticmethod
    def from_npz(file_name: str, layer_num: int, num_attention_heads: int, device: Optional[torch.device] = None, dtype=None):
        return BertLayer(BertAttention.from_npz(file_name, layer_num, num_attention_heads, device, dtype),
                         BertIntermediate.from_npz(file_name, layer_num, device, dtype),
                         BertOutput.from_npz(file_name, layer_num, device, dtype))


class BertEncoder:
    def __init__(self, layer: Sequence[BertLayer]):
        self.layer = layer

    def __call__(self, hidden_states: AnyTensor, attention_mask: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 output_attentions: Optional[bool] = False, output_hidden_states: Optional[bool] = False,
                 return_type: Optional[ReturnType] = None):
        all_hidden_states, all_attentions = (), ()
        hidden_states = try_convert(hidden_states)
        attention_mask = try_convert(attention_mask)
        for l in self.layer:
            layer_outputs = l(hidden_states=hidden_states, attention_mask=attention_mask, output_attentions=output_attentions,
                              return_type=ReturnType.turbo_transformers)
            if output_hidden_states:
                all_hidden_states = all_hidden_states + (hidden_states, )
            hidden_states = layer_outputs[0]
            if output_attentions:
                all_attentions = all_attentions + (layer_outputs[1], )
        outputs = (convert_returns_as_type(hidden_states, return_type), )
        # As in the reference, the last hidden state is outputs[0] only: one storage cannot be exported twice.
        if output_hidden_states:
            outputs = outputs + (all_hidden_states, )
        if output_attentions:
            outputs = outputs + (all_attentions, )
        return outputs

    @staticmethod
    def from_torch(encoder):
        return BertEncoder([BertLayer.from_torch(l) for l in encoder.layer])

    @staticmethod
    def from_npz(file_name: str, num_hidden_layers: int, num_attention_heads: int, device: Optional[torch.device] = None,
                 dtype=None):
        return BertEncoder([BertLayer.from_npz(file_name, i, num_attention_heads, device, dtype) for i in range(num_hidden_layers)])


class SequencePool(cxx.SequencePool):
    def __call__(self, input_tensor: AnyTensor, return_type: Optional[ReturnType] = None,
                 output_tensor: Optional[cxx.Tensor] = None):
        input_tensor = try_convert(input_tensor)
        output_tensor = create_empty_if_none(output_tensor)
        super().__call__(input_tensor, output_tensor)
        return convert_returns_as_type(output_tensor, return_type)


class PoolingType(enum.Enum):
    FIRST = "First"
    LAST = "Last"
    MEAN = "Mean"
    MAX = "Max"


PoolingMap = {PoolingType.FIRST: "First", PoolingType.LAST: "Last", PoolingType.MEAN: "Mean", PoolingType.MAX: "Max"}


class BertPooler(cxx.BertPooler):
    def __call__(self, input_tensor: AnyTensor, return_type: Optional[ReturnType] = None, output: Optional[cxx.Tensor] = None):
        input_tensor = try_convert(input_tensor)
        output = create_empty_if_none(output)
        super().__call__(input_tensor, output)
        return convert_returns_as_type(output, return_type)

    @staticmethod
    def from_torch(pooler):
        p = to_param_dict(pooler)
        return BertPooler(convert2tt_tensor(_t(p['dense.weight'])), convert2tt_tensor(p['dense.bias']))

    @staticmethod
    def from_npz(file_name: str, device: Optional[torch.device] = None, dtype=None):
        f = np.load(file_name)
        return BertPooler(_npz(f, 'pooler.dense.weight', device, dtype), _npz(f, 'pooler.dense.bias', device, dtype))


def _require_cuda(model, device):
    if device is None:
        device = next(model.parameters()).device
    device = torch.device(device)
    if device.type != 'cuda':
        raise RuntimeError("this runtime computes on CUDA devices only (no CPU path): pass a cuda device")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available")
    model.to(device)
    return device


class BertModelNoPooler:
    def __init__(self, embeddings: BertEmbeddings, encoder: BertEncoder):
        self.embeddings = embeddings
        self.encoder = encoder
        self.prepare = cxx.PrepareBertMasks()

    def __call__(self, inputs: AnyTensor, attention_masks: Optional[AnyTensor] = None, token_type_ids: Optional[AnyTensor] = None,
                 position_ids: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 inputs_embeds: Optional[AnyTensor] = None, output_attentions: Optional[bool] = None,
                 output_hidden_states: Optional[bool] = None, pooling_type: PoolingType = PoolingType.FIRST,
                 return_type: Optional[ReturnType] = None):
        use_current_stream(inputs if isinstance(inputs, torch.Tensor) else None)
        no_mask = attention_masks is None
        attention_masks = try_convert(create_empty_if_none(attention_masks))
        token_type_ids = try_convert(create_empty_if_none(token_type_ids))
        position_ids = try_convert(create_empty_if_none(position_ids))
        inputs = try_convert(inputs)
        extended_attention_masks = cxx.Tensor.create_empty()
        self.prepare(inputs, attention_masks, token_type_ids, position_ids, extended_attention_masks)
        hidden_cache = self.embeddings(inputs, position_ids=position_ids, token_type_ids=token_type_ids,
                                       return_type=ReturnType.turbo_transformers)
        # Without a caller mask the additive mask is all zeros: 16-bit models then run the mask-free attention kernel
        # (fp32 models keep the reference's sequence, mask included).
        if no_mask and hidden_cache.dtype() in ("float16", "bfloat16"):
            extended_attention_masks = None
        return self.encoder(hidden_states=hidden_cache, attention_mask=extended_attention_masks,
                            output_attentions=output_attentions, output_hidden_states=output_hidden_states,
                            return_type=return_type)

    @staticmethod
    def from_torch(model, device: Optional[torch.device] = None):
        _require_cuda(model, device)
        return BertModelNoPooler(BertEmbeddings.from_torch(model.embeddings), BertEncoder.from_torch(model.encoder))

    @staticmethod
    def from_npz(file_name: str, config, device: Optional[torch.device] = None, dtype=None):
        return BertModelNoPooler(BertEmbeddings.from_npz(file_name, device, dtype),
                                 BertEncoder.from_npz(file_name, config.num_hidden_layers, config.num_attention_heads, device, dtype))


class BertModel:
    """`backend` is kept for call compatibility; only "turbo" (this runtime) exists. The reference's
    onnxruntime backend is not provided: asking for it raises instead of silently switching engines."""

    def __init__(self, model, pooler=None, backend="turbo", config=None):
        if backend != "turbo":
            raise NotImplementedError("only the 'turbo' backend exists in this runtime")
        self.backend = "turbo"
        self.config = config
        self.bertmodel_nopooler = model
        self.pooler = pooler

    def __call__(self, inputs: AnyTensor, attention_masks: Optional[AnyTensor] = None, token_type_ids: Optional[AnyTensor] = None,
                 position_ids: Optional[AnyTensor] = None, head_mask: Optional[AnyTensor] = None,
                 inputs_embeds: Optional[AnyTensor] = None, output_attentions: Optional[bool] = None,
                 output_hidden_states: Optional[bool] = None, pooling_type: PoolingType = PoolingType.FIRST,
                 pooler_output: Optional[AnyTensor] = None, return_type: Optional[ReturnType] = None):
        encoder_outputs = self.bertmodel_nopooler(inputs, attention_masks, token_type_ids, position_ids,
                                                  inputs_embeds=inputs_embeds, output_attentions=output_attentions,
                                                  output_hidden_states=output_hidden_states, pooling_type=pooling_type,
                                                  return_type=ReturnType.turbo_transformers)
        sequence_output = encoder_outputs[0]
        self.seq_pool = SequencePool(PoolingMap[pooling_type])
        sequence_pool_output = self.seq_pool(input_tensor=sequence_output, return_type=ReturnType.turbo_transformers)
        pooler_output = self.pooler(sequence_pool_output, return_type, pooler_output)
        return (convert_returns_as_type(sequence_output, return_type), pooler_output) + encoder_outputs[1:]

    @staticmethod
    def from_torch(model, device: Optional[torch.device] = None, backend: Optional[str] = None, use_memory_opt=False):
        """model: a HuggingFace BertModel (fp32, fp16 or bf16); device: a CUDA device.
        use_memory_opt reserves the activation arena of the first call's shape in the device pool."""
        if backend not in (None, "turbo"):
            raise NotImplementedError("only the 'turbo' backend exists in this runtime (no onnxruntime dispatch)")
        _require_cuda(model, device)
        nopooler = BertModelNoPooler(BertEmbeddings.from_torch(model.embeddings), BertEncoder.from_torch(model.encoder))
        return BertModel(nopooler, BertPooler.from_torch(model.pooler), "turbo", model.config)

    @staticmethod
    def from_pretrained(model_id_or_path: str, device: Optional[torch.device] = None, backend: Optional[str] = None):
        from transformers.models.bert.modeling_bert import BertModel as TorchBertModel
        torch_model = TorchBertModel.from_pretrained(model_id_or_path)
        model = BertModel.from_torch(torch_model, device, backend)
        model.config = torch_model.config
        model._torch_model = torch_model  # keeps the aliased weights alive
        return model

    @staticmethod
    def from_npz(file_name: str, config, device: Optional[torch.device] = None, dtype=None):
        return BertModel(BertModelNoPooler.from_npz(file_name, config, device, dtype), BertPooler.from_npz(file_name, device, dtype),
                         backend="turbo", config=config)
