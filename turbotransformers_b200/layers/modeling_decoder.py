"""TransformerDecoderLayer and TransformerDecoder with the call signatures of the reference's
python/turbo_transformers/layers/modeling_decoder.py:42-356 (the OpenNMT-py transformer decoder): pre-LN self attention with
a residual, pre-LN context attention over the encoder memory with a residual, feed-forward block.

`from_onmt` reads attribute and parameter names only (self_attn, context_attn, feed_forward, layer_norm_1, layer_norm_2;
linear_keys / linear_values / linear_query / final_linear; w_1 / w_2 / layer_norm), so any module laid out like OpenNMT-py's
works; OpenNMT-py itself is not needed.

Stepwise decoding (`step` given) keeps four cache entries per layer: "memory_keys" / "memory_values" (the projected encoder
memory, computed at the first step) for every dtype, and "self_keys" / "self_values" (appended in place) for 16-bit models
with 64-wide heads.
"""
from typing import Optional, Sequence

import torch

from .._cxx import cxx
from .modules import MultiHeadedAttention, PositionwiseFeedForward
from .return_type import ReturnType, convert_returns_as_type
from .utils import create_empty_if_none, try_convert

__all__ = ['TransformerDecoderLayer', 'TransformerDecoder']


class TransformerDecoderLayer:
    def __init__(self, self_attn: MultiHeadedAttention, context_attn: MultiHeadedAttention, feed_forward: PositionwiseFeedForward):
        if not isinstance(self_attn, MultiHeadedAttention):
            raise TypeError("self_attn should be of type MultiHeadedAttention")
        if not isinstance(context_attn, MultiHeadedAttention):
            raise TypeError("context_attn should be of type MultiHeadedAttention")
        self.self_attn, self.context_attn, self.feed_forward = self_attn, context_attn, feed_forward

    def __call__(self, input_tensor: torch.Tensor, memory_bank: torch.Tensor, src_pad_mask: torch.Tensor, tgt_pad_mask: torch.Tensor,
                 layer_cache: Optional[dict] = None, step: Optional[int] = None, future: Optional[bool] = False,
                 with_align: Optional[bool] = False, return_type: Optional[ReturnType] = None, output: Optional[cxx.Tensor] = None):
        """input_tensor [B, T, H], memory_bank [B, src_len, H], src_pad_mask [B, 1, src_len] and tgt_pad_mask [B, 1, T]
        (true / 1 = padding). Returns (output [B, T, H], context attention of head 0 [B, T, src_len], None)."""
        if with_align:
            raise ValueError("with_align must be False")
        src_mask = src_pad_mask.float() * -1e18
        dec_mask = None
        if step is None:
            tgt_len = tgt_pad_mask.size(-1)
            if not future:  # padding + future positions, [B, T, T]
                future_mask = torch.ones([tgt_len, tgt_len], device=tgt_pad_mask.device, dtype=torch.float32).triu_(1)
                dec_mask = torch.gt(tgt_pad_mask.float() + future_mask.view(1, tgt_len, tgt_len), 0).float()
            else:           # padding only, [B, 1, T]
                dec_mask = tgt_pad_mask.float()
            dec_mask = (dec_mask * -1e18).contiguous()
        query, _ = self.self_attn(input_tensor, input_tensor, input_tensor, mask=dec_mask, layer_cache=layer_cache, attn_type="self",
                                  pre_layernorm=True, post_add_input=True, return_type=ReturnType.turbo_transformers)
        mid, attns = self.context_attn(memory_bank, memory_bank, query, mask=src_mask.contiguous(), layer_cache=layer_cache,
                                       attn_type="context", pre_layernorm=True, post_add_input=True,
                                       return_type=ReturnType.turbo_transformers, output_attentions=True)
        out = self.feed_forward(mid, return_type=return_type, is_trans_weight=self._ffn_trans, output=output)
        return out, convert_returns_as_type(attns, ReturnType.TORCH)[:, 0, :, :].contiguous(), None

    _ffn_trans = True

    @staticmethod
    def from_onmt(transformer_decoder_layer):
        self_attn = MultiHeadedAttention.from_onmt(transformer_decoder_layer.self_attn, transformer_decoder_layer.layer_norm_1)
        context_attn = MultiHeadedAttention.from_onmt(transformer_decoder_layer.context_attn, transformer_decoder_layer.layer_norm_2)
        feed_forward = PositionwiseFeedForward.from_onmt(transformer_decoder_layer.feed_forward)
        eps = float(getattr(transformer_decoder_layer.layer_norm_1, "eps", 1e-6))
        self_attn.set_pre_layernorm_eps(eps)
        context_attn.set_pre_layernorm_eps(eps)
        feed_forward.set_layernorm_eps(float(getattr(transformer_decoder_layer.feed_forward.layer_norm, "eps", 1e-6)))
        return TransformerDecoderLayer(self_attn, context_attn, feed_forward)


class TransformerDecoder:
    """The decoder stack: the embeddings and the final LayerNorm stay torch modules, as in the reference
    (modeling_decoder.py:230-329); tensors are time-major at this interface ([len, batch, ...]) like OpenNMT-py's."""

    def __init__(self, embeddings, transformer_layers: Sequence[TransformerDecoderLayer], layer_norm: torch.nn.Module,
                 copy_attn: Optional[bool] = False, alignment_layer: Optional[int] = 0):
        self.embeddings, self.transformer_layers, self.layer_norm = embeddings, list(transformer_layers), layer_norm
        self._copy, self.alignment_layer = copy_attn, alignment_layer
        self.state = {}

    def init_state(self, src, memory_bank, enc_hidden):
        self.state["src"] = src
        self.state["cache"] = None

    def _init_cache(self, memory_bank):
        self.state["cache"] = {f"layer_{i}": {"memory_keys": None, "memory_values": None, "self_keys": None, "self_values": None}
                               for i in range(len(self.transformer_layers))}

    def __call__(self, tgt: torch.Tensor, memory_bank: torch.Tensor, step: Optional[int] = None, **kwargs):
        """tgt [tgt_len, B, 1] token ids, memory_bank [src_len, B, H], memory_lengths=[B]. Returns (dec_outs [tgt_len, B, H],
        {"std": attention [tgt_len, B, src_len]})."""
        if step == 0:
            self._init_cache(memory_bank)
        if kwargs.pop('with_align', False):
            raise ValueError("with_align must be False")
        tgt_words = tgt[:, :, 0].transpose(0, 1)
        emb = self.embeddings(tgt, step=step)
        assert emb.dim() == 3  # len x batch x embedding_dim
        output = emb.transpose(0, 1).contiguous()
        src_memory_bank = memory_bank.transpose(0, 1).contiguous()
        src_lens = kwargs["memory_lengths"]
        src_max_len = self.state["src"].shape[0]
        src_pad_mask = ~(torch.arange(src_max_len, device=src_lens.device)[None, :] < src_lens[:, None]).unsqueeze(1)
        tgt_pad_mask = tgt_words.data.eq(self.embeddings.word_padding_idx).unsqueeze(1)  # [B, 1, T_tgt]
        attn = None
        for i, layer in enumerate(self.transformer_layers):
            layer_cache = self.state["cache"][f"layer_{i}"] if step is not None else None
            output, attn, _ = layer(output, src_memory_bank, src_pad_mask, tgt_pad_mask, layer_cache=layer_cache, step=step)
        output = self.layer_norm(output)
        attns = {"std": attn.transpose(0, 1).contiguous()}
        if self._copy:
            attns["copy"] = attns["std"]
        return output.transpose(0, 1).contiguous(), attns

    @staticmethod
    def from_onmt(model, device: Optional[torch.device] = None):
        if device is not None and 'cuda' in device.type and torch.cuda.is_available():
            model.to(device)
        layers = [TransformerDecoderLayer.from_onmt(layer) for layer in model.transformer_layers]
        return TransformerDecoder(model.embeddings, layers, model.layer_norm, getattr(model, "_copy", False),
                                  getattr(model, "alignment_layer", 0))
