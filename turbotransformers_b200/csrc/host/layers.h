// Layer classes with the names, constructor argument order and operator() signatures of the reference's
// turbo_transformers/layers/*.h, re-implemented over the C ABI in include/ttb.h.
//
//   fp32 tensors  -> the reference's own op sequence on exact-precision kernels (MatMul, SplitAddBias...,
//                    BatchMatMul, ApplyMaskAndSoftmax, ..., AddBiasLayerNorm), scores materialised
//   fp16 / bf16   -> tcgen05 GEMMs with fused epilogues + one attention kernel over packed tokens
//   int8          -> (after QuantizeInt8()) int8 tcgen05 GEMMs with dequantising epilogues
// The dtype is taken from the weights handed to the constructor; activations must match it.
// No layer keeps per-call state in members (what a call does follows from its arguments alone), so one object may be
// called from several host threads (the reference serialised MultiHeadedAttention behind a global mutex).
#pragma once
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "core.h"

namespace turbo_transformers {
namespace layers {

// A Linear weight plus its lazily-built tensor-core re-layouts. The source tensor may alias memory owned
// by the caller's framework and is never written.
class PackedLinear {
 public:
  PackedLinear() : weight_(nullptr), bias_(nullptr) {}
  PackedLinear(core::Tensor weight, core::Tensor bias) : weight_(std::move(weight)), bias_(std::move(bias)) {}
  PackedLinear(PackedLinear&&) = default;
  const core::Tensor& weight() const { return weight_; }
  const core::Tensor& bias() const { return bias_; }
  int64_t in_dim(bool is_trans) const { return weight_.shape(is_trans ? 1 : 0); }
  int64_t out_dim(bool is_trans) const { return weight_.shape(is_trans ? 0 : 1); }
  // K-major [N,K] copy in the weight's own 16-bit dtype (built on first use).
  const void* Packed(bool is_trans) const;
  // fp32 weights as two tf32 planes [2][N,K] (hi, then lo), for the three-product tensor-core GEMM.
  const float* PackedTf32(bool is_trans) const;
  // int8 [N,K] copy + device scale (built on first use); `col_sum` (may be null) selects the reference recipe's
  // quantiser (torch's per-tensor rule) and receives the per-output-row sums its zero-point correction needs.
  void Int8(bool is_trans, const int8_t** wq, const float** scale, const int32_t** col_sum = nullptr) const;
  // The bias as fp32 (for GEMMs that write an fp32 residual stream).
  const float* BiasF32() const;
  // kInt8PerRow: the benchmark's scheme (per-row symmetric activations); kInt8Reference: the reference's recipe
  // (qmodeling_bert.py:13-45: torch dynamic quantisation, per-tensor affine 7-bit activations).
  enum Int8Mode { kInt8Off = 0, kInt8PerRow = 1, kInt8Reference = 2 };
  void set_int8(bool on) { int8_mode_ = on ? kInt8PerRow : kInt8Off; }
  void set_int8_mode(int mode) { int8_mode_ = mode; }
  bool use_int8() const { return int8_mode_ != kInt8Off; }
  int int8_mode() const { return int8_mode_; }

  // out[M,N] = epilogue(x[M,K] . W + bias); picks the kernel by dtype / int8 mode.
  // `ldo` (elements between output rows) defaults to N. A bf16 x that carries a lo plane is used at full precision
  // (two passes). out_lo (bf16 only) receives the second plane of the output. f32_out: `out` and `residual` are fp32
  // (the residual stream of a bf16 model in its precise mode).
  // out = LayerNorm(x . W + bias + residual) * gamma + beta: one kernel for the plain 16-bit product where the shape allows
  // it, else Forward with the residual epilogue followed by the layer norm kernel.
  void ForwardLayerNorm(const core::Tensor& x, int64_t M, const void* residual, const core::Tensor& gamma, const core::Tensor& beta, float eps,
                        void* out, bool is_trans, const char* name) const;
  // q8_of_out (per-row int8 mode): the tensor that owns `out`; it gets the int8 form of the output attached (q8(), q8_scale()).
  void Forward(const core::Tensor& x, int64_t M, int epilogue, const void* residual, void* out, bool is_trans,
               const char* name, int64_t ldo = 0, void* out_lo = nullptr, bool f32_out = false, core::Tensor* q8_of_out = nullptr) const;

 private:
  core::Tensor weight_, bias_;
  int int8_mode_ = kInt8Off;
  struct Cache {
    std::mutex mu;
    core::Tensor packed[2]{core::Tensor(nullptr), core::Tensor(nullptr)};
    core::Tensor tf32[2]{core::Tensor(nullptr), core::Tensor(nullptr)};
    core::Tensor q[2]{core::Tensor(nullptr), core::Tensor(nullptr)};
    core::Tensor qscale[2]{core::Tensor(nullptr), core::Tensor(nullptr)};
    core::Tensor qref[2]{core::Tensor(nullptr), core::Tensor(nullptr)};
    core::Tensor qref_scale[2]{core::Tensor(nullptr), core::Tensor(nullptr)};
    core::Tensor qref_colsum[2]{core::Tensor(nullptr), core::Tensor(nullptr)};
    core::Tensor bias_f32{nullptr};
  };
  std::unique_ptr<Cache> cache_{new Cache()};
};

class BERTEmbedding {
 public:
  BERTEmbedding(core::Tensor word_embeddings, core::Tensor position_embeddings, core::Tensor token_type_embeddings,
                core::Tensor layer_norm_weights, core::Tensor layer_norm_bias, float dropout_rate = 0.f)
      : word_embedings_(std::move(word_embeddings)), position_embeddings_(std::move(position_embeddings)),
        token_type_embeddings_(std::move(token_type_embeddings)), layer_norm_weights_(std::move(layer_norm_weights)),
        layer_norm_bias_(std::move(layer_norm_bias)) {
    EnforceShapeAndType();
  }
  void EnforceShapeAndType() const;
  void operator()(const core::Tensor& input_ids, const core::Tensor& position_ids, const core::Tensor& token_type_ids,
                  core::Tensor* output_tensor) const;
  // Packed variable-length form: ids [sumL]; positions restart at 0 per sequence and types are 0 unless packed
  // position_ids / token_type_ids ([sumL], null tensors = defaults) are given.
  void Packed(const core::Tensor& input_ids, const std::vector<int64_t>& seq_lens, core::Tensor* output_tensor,
              const core::Tensor& position_ids = core::Tensor(nullptr), const core::Tensor& token_type_ids = core::Tensor(nullptr)) const;

 private:
  core::Tensor word_embedings_, position_embeddings_, token_type_embeddings_, layer_norm_weights_, layer_norm_bias_;
};

class MultiHeadedAttention {
 public:
  MultiHeadedAttention(core::Tensor k_weight, core::Tensor k_bias, core::Tensor v_weight, core::Tensor v_bias,
                       core::Tensor q_weight, core::Tensor q_bias, core::Tensor dense_weight, core::Tensor dense_bias,
                       core::Tensor qkv_weight, core::Tensor qkv_bias, int64_t num_attention_heads);
  MultiHeadedAttention(core::Tensor k_weight, core::Tensor k_bias, core::Tensor v_weight, core::Tensor v_bias,
                       core::Tensor q_weight, core::Tensor q_bias, core::Tensor dense_weight, core::Tensor dense_bias,
                       core::Tensor qkv_weight, core::Tensor qkv_bias, core::Tensor layernorm_gamma,
                       core::Tensor layernorm_beta, int64_t num_attention_heads);
  void EnforceShapeAndType() const;

  void operator()(const core::Tensor& key_tensor, const core::Tensor& value_tensor, const core::Tensor& query_tensor,
                  const core::Tensor& attention_mask, const std::string& attn_type, core::Tensor* output,
                  core::Tensor* att_score, std::unordered_map<std::string, core::Tensor*> layer_cache,
                  bool pre_layernorm = false, bool post_layernorm = false, bool post_add_input = false,
                  bool is_trans_weight = false) const;

  // Shared implementation: seq_lens == nullptr means a [B,L,H] batch of equal lengths, otherwise
  // query_tensor is packed [1,sumL,H].
  // cache_keys / cache_values (both or neither): the decoder's `layer_cache["self_keys" / "self_values"]`: tensors whose shape
  // reads [T, B, H] (paged buffers underneath) and that this call grows by the query's tokens (16-bit models, equal-length
  // batches).
  void Run(const core::Tensor& query_tensor, const core::Tensor& attention_mask, const std::vector<int64_t>* seq_lens,
           core::Tensor* output, core::Tensor* att_score, bool pre_layernorm, bool post_layernorm, bool post_add_input,
           bool is_trans_weight, core::Tensor* cache_keys = nullptr, core::Tensor* cache_values = nullptr) const;

  // `att_score` is a per-call choice: a 16-bit model given nullptr skips the [B,heads,L,L] score tensor (the largest HBM
  // round trip of the reference path) and runs the fused attention kernel; given a tensor it materialises the scores into
  // it as the reference does. fp32 models always materialise (into a temporary when att_score is nullptr).
  void set_pre_layernorm_eps(float eps) { pre_ln_eps_ = eps; }  // the reference hard-codes 1e-6
  void set_causal(bool on) { causal_ = on; }                    // decoder-style self-attention without a mask tensor
  void QuantizeInt8() { qkv_.set_int8(true); dense_.set_int8(true); }
  int64_t num_attention_heads() const { return num_attention_heads_; }

 protected:
  // attn_type == "context" (encoder-decoder attention, multi_headed_attention.cpp:45-167 of the reference): queries from
  // query_tensor [B, Lq, H], keys / values from key_tensor / value_tensor [B, Lk, H] or, once computed, from
  // layer_cache["memory_keys" / "memory_values"] ([B, heads, Lk, d], the reference's layout).
  // q_lens / k_lens (both or neither): the packed form of MultiHeadedAttentionSmartBatch, query_tensor [1, sum(q_lens), H]
  // and key_tensor / value_tensor [1, sum(k_lens), H] (multi_headed_attention_smart_batch.cpp:34-170).
  void RunContext(const core::Tensor& key_tensor, const core::Tensor& value_tensor, const core::Tensor& query_tensor,
                  const core::Tensor& attention_mask, core::Tensor* output, core::Tensor* att_score, core::Tensor* memory_keys,
                  core::Tensor* memory_values, bool pre_layernorm, bool post_layernorm, bool post_add_input,
                  bool is_trans_weight, const std::vector<int64_t>* q_lens = nullptr,
                  const std::vector<int64_t>* k_lens = nullptr) const;
  // Output projection of the token-major attention result [T, H] and what follows it (residual, layer norm).
  void Finish(const core::Tensor& context, const core::Tensor& x, int64_t T, core::Tensor* output, bool post_layernorm,
              bool post_add_input, bool is_trans_weight) const;

  PackedLinear k_, v_, q_;  // separate projections: context attention only
  PackedLinear qkv_, dense_;
  core::Tensor layernorm_gamma_, layernorm_beta_;
  int64_t num_attention_heads_;
  bool causal_ = false;
  float pre_ln_eps_ = 1e-6f;
};

class MultiHeadedAttentionSmartBatch : public MultiHeadedAttention {
 public:
  using MultiHeadedAttention::MultiHeadedAttention;
  void operator()(const core::Tensor& key_tensor, const core::Tensor& value_tensor, const core::Tensor& query_tensor,
                  const core::Tensor& attention_mask, const std::string& attn_type, core::Tensor* output,
                  core::Tensor* att_score, std::unordered_map<std::string, core::Tensor*> layer_cache,
                  const std::vector<int64_t>& query_seq_len_list, const std::vector<int64_t>& key_seq_len_list,
                  bool pre_layernorm = false, bool post_layernorm = false, bool post_add_input = false,
                  bool is_trans_weight = false) const;
};

class BertAttention : public MultiHeadedAttention {
 public:
  BertAttention(core::Tensor qkv_weight, core::Tensor qkv_bias, core::Tensor dense_weight, core::Tensor dense_bias,
                core::Tensor layer_norm_weight, core::Tensor layer_norm_bias, int64_t num_attention_heads)
      : MultiHeadedAttention(core::Tensor(nullptr), core::Tensor(nullptr), core::Tensor(nullptr), core::Tensor(nullptr),
                             core::Tensor(nullptr), core::Tensor(nullptr), std::move(dense_weight), std::move(dense_bias),
                             std::move(qkv_weight), std::move(qkv_bias), std::move(layer_norm_weight),
                             std::move(layer_norm_bias), num_attention_heads) {}
  void operator()(const core::Tensor& input_tensor, const core::Tensor& attention_mask, core::Tensor* output,
                  core::Tensor* attn = nullptr, bool is_trans_weight = false) const;
};

class BertIntermediate {
 public:
  BertIntermediate(core::Tensor dense_weight, core::Tensor dense_bias) : dense_(std::move(dense_weight), std::move(dense_bias)) {
    EnforceShapeAndType();
  }
  void EnforceShapeAndType() const;
  void operator()(const core::Tensor& input_tensor, core::Tensor* output_tensor) const;
  void QuantizeInt8(int mode = PackedLinear::kInt8PerRow) { dense_.set_int8_mode(mode); }

 private:
  PackedLinear dense_;
};

class BertOutput {
 public:
  BertOutput(core::Tensor dense_weight, core::Tensor dense_bias, core::Tensor layer_norm_weight, core::Tensor layer_norm_bias)
      : dense_(std::move(dense_weight), std::move(dense_bias)), layer_norm_weight_(std::move(layer_norm_weight)),
        layer_norm_bias_(std::move(layer_norm_bias)) {
    EnforceShapeAndType();
  }
  void EnforceShapeAndType() const;
  void operator()(const core::Tensor& hidden_states, const core::Tensor& input_tensor, core::Tensor* output_tensor) const;
  void QuantizeInt8(int mode = PackedLinear::kInt8PerRow) { dense_.set_int8_mode(mode); }

 private:
  PackedLinear dense_;
  core::Tensor layer_norm_weight_, layer_norm_bias_;
};

class BertPooler {
 public:
  BertPooler(core::Tensor dense_weight, core::Tensor dense_bias) : dense_(std::move(dense_weight), std::move(dense_bias)) {
    EnforceShapeAndType();
  }
  void EnforceShapeAndType() const;
  void operator()(const core::Tensor& input_tensor, core::Tensor* output_tensor) const;

 private:
  PackedLinear dense_;
};

class SequencePool {
 public:
  explicit SequencePool(const std::string& pool_type);
  void operator()(const core::Tensor& input, core::Tensor* output) const;
  // First/Last/Mean/Max per sequence of a packed [1,sumL,H] tensor -> [B,H].
  void Packed(const core::Tensor& input, const std::vector<int64_t>& seq_lens, core::Tensor* output) const;

 private:
  int pool_type_;
};

class PrepareBertMasks {
 public:
  void operator()(const core::Tensor& inputs, core::Tensor* att_mask, core::Tensor* seq_type, core::Tensor* position_ids,
                  core::Tensor* extended_attention_mask) const;
};

// Pre-LN feed-forward block: out = x + W2 act(W1 LN(x) + b1) + b2 (positionwise_ffn.cpp:31-75).
// The reference's activation is ReLU; "gelu" selects the tanh-form GELU for GPT-2 style blocks.
class PositionwiseFeedForward {
 public:
  PositionwiseFeedForward(core::Tensor dense_weight_1, core::Tensor dense_bias_1, core::Tensor dense_weight_2,
                          core::Tensor dense_bias_2, core::Tensor layer_norm_weight, core::Tensor layer_norm_bias)
      : dense1_(std::move(dense_weight_1), std::move(dense_bias_1)), dense2_(std::move(dense_weight_2), std::move(dense_bias_2)),
        layer_norm_weight_(std::move(layer_norm_weight)), layer_norm_bias_(std::move(layer_norm_bias)) {}
  void operator()(const core::Tensor& input_tensor, core::Tensor* output, bool is_trans_weight = true) const;
  void set_activation(const std::string& act);
  void set_layernorm_eps(float eps) { eps_ = eps; }

 private:
  PackedLinear dense1_, dense2_;
  core::Tensor layer_norm_weight_, layer_norm_bias_;
  int act_ = TTB_ACT_RELU;
  float eps_ = 1e-12f;
};

// Post-LN feed-forward block of DistilBERT (positionwise_ffn.cpp:79-123): out = LN(x + W2 gelu(W1 x + b1) + b2), eps 1e-12.
// The same two fused GEMMs and LayerNorm as BertIntermediate + BertOutput.
class DistrillFFN {
 public:
  DistrillFFN(core::Tensor dense_weight_1, core::Tensor dense_bias_1, core::Tensor dense_weight_2, core::Tensor dense_bias_2,
              core::Tensor layer_norm_weight, core::Tensor layer_norm_bias)
      : dense1_(std::move(dense_weight_1), std::move(dense_bias_1)), dense2_(std::move(dense_weight_2), std::move(dense_bias_2)),
        layer_norm_weight_(std::move(layer_norm_weight)), layer_norm_bias_(std::move(layer_norm_bias)) {}
  void operator()(const core::Tensor& input_tensor, core::Tensor* output, bool is_trans_weight = true) const;

 private:
  PackedLinear dense1_, dense2_;
  core::Tensor layer_norm_weight_, layer_norm_bias_;
};

// Feed-forward half of an ALBERT layer (albert_layer.cpp:31-50): hidden_output = gelu(x W1 + b1),
// output = LN(x + hidden_output W2 + b2). Weights are [in, out].
class AlbertLayer {
 public:
  AlbertLayer(core::Tensor dense_weight, core::Tensor dense_bias, core::Tensor dense_output_weight, core::Tensor dense_output_bias,
              core::Tensor layer_norm_weight, core::Tensor layer_norm_bias)
      : dense_(std::move(dense_weight), std::move(dense_bias)), dense_output_(std::move(dense_output_weight), std::move(dense_output_bias)),
        layer_norm_weight_(std::move(layer_norm_weight)), layer_norm_bias_(std::move(layer_norm_bias)) {
    EnforceShapeAndType();
  }
  void EnforceShapeAndType() const;
  void operator()(const core::Tensor& input_tensor, core::Tensor* hidden_output, core::Tensor* output) const;

 private:
  PackedLinear dense_, dense_output_;
  core::Tensor layer_norm_weight_, layer_norm_bias_;
};

// In-place bias + tanh-GELU on a projection computed elsewhere (layers/addbias_act.cpp:20-23).
class FusedAddBiasGELU {
 public:
  explicit FusedAddBiasGELU(core::Tensor bias) : bias_(std::move(bias)) {}
  void operator()(core::Tensor* input_tensor) const;

 private:
  core::Tensor bias_;
};

// In-place out = LN(out + input + bias) (layers/addbias_layernorm.cpp:20-24).
class FusedAddBiasLayerNorm {
 public:
  FusedAddBiasLayerNorm(core::Tensor bias, core::Tensor norm_weight, core::Tensor norm_bias)
      : bias_(std::move(bias)), norm_weight_(std::move(norm_weight)), norm_bias_(std::move(norm_bias)) {}
  void operator()(const core::Tensor& input_tensor, core::Tensor* output_tensor) const;

 private:
  core::Tensor bias_, norm_weight_, norm_bias_;
};

// Stand-alone LayerNorm (kernels::LayerNorm, layer_norm.cpp:32-91) for pre-LN models' final norm.
class LayerNorm {
 public:
  LayerNorm(core::Tensor gamma, core::Tensor beta, float eps) : gamma_(std::move(gamma)), beta_(std::move(beta)), eps_(eps) {}
  void operator()(const core::Tensor& input, core::Tensor* output) const;

 private:
  core::Tensor gamma_, beta_;
  float eps_;
};

// Token + learned position embedding without a layer norm (decoder-only models): two
// kernels::LookupEmbedding passes (embedding.cpp:28-85), set then accumulate.
class TokenPositionEmbedding {
 public:
  TokenPositionEmbedding(core::Tensor token_table, core::Tensor position_table)
      : token_(std::move(token_table)), position_(std::move(position_table)) {}
  // ids [B,L] -> [B,L,H], positions position_offset .. position_offset+L-1 (the offset is the cached length when decoding)
  void operator()(const core::Tensor& input_ids, core::Tensor* output, int64_t position_offset = 0) const;

 private:
  core::Tensor token_, position_;
};

// out = x . W (+ bias): kernels::MatMul as a layer, used for the tied-embedding logits of decoder models.
class Linear {
 public:
  Linear(core::Tensor weight, core::Tensor bias, bool is_trans_weight)
      : dense_(std::move(weight), std::move(bias)), is_trans_(is_trans_weight) {}
  void operator()(const core::Tensor& input, core::Tensor* output) const;
  // The same product with the output's last dimension rounded up to a multiple of 8 elements (rows that start on 16-byte
  // boundaries, which the tensor-core epilogue stores at full speed): output is [..., PaddedWidth()], of which the first
  // out-features columns are the result and the rest is undefined. For widths like a 50257-entry vocabulary, where
  // operator() pays a second pass over the output to compact the rows.
  void Padded(const core::Tensor& input, core::Tensor* output) const;
  int64_t Width() const { return dense_.out_dim(is_trans_); }
  int64_t PaddedWidth() const { return (Width() + 7) / 8 * 8; }

 private:
  PackedLinear dense_;
  bool is_trans_;
};

}  // namespace layers
}  // namespace turbo_transformers
