#include "layers.h"

#include <algorithm>
#include <cmath>

namespace turbo_transformers {
namespace layers {

using core::Check;
using core::DeviceContext;
using core::Tensor;

namespace {

// dtype of a floating tensor as ttb_dtype; throws for anything else or for host memory.
int FloatType(const Tensor& t, const char* what) {
  TT_ENFORCE(!t.is_null(), "%s is null", what);
  if (!t.on_gpu()) TT_THROW("%s is not on a CUDA device: this runtime has no CPU path", what);
  int dt = core::ToTTBDtype(t.dtype());
  TT_ENFORCE(dt == TTB_F32 || dt == TTB_F16 || dt == TTB_BF16, "%s must be fp32, fp16 or bf16", what);
  return dt;
}

void SameTypeDevice(const Tensor& a, const Tensor& b, const char* what) {
  TT_ENFORCE(core::SameType(a.dtype(), b.dtype()), "%s: tensors differ in dtype", what);
  TT_ENFORCE(a.device_type() == b.device_type() && a.device_id() == b.device_id(), "%s: tensors are on different devices", what);
}

std::vector<int64_t> ShapeOf(const Tensor& t) {
  std::vector<int64_t> s(t.n_dim());
  for (size_t i = 0; i < s.size(); ++i) s[i] = t.shape((int)i);
  return s;
}

std::vector<int64_t> WithLast(const Tensor& t, int64_t last) {
  auto s = ShapeOf(t);
  s.back() = last;
  return s;
}

// bf16 models in their precise mode: activations travel as a bf16 value plus a lo plane (what the rounding dropped) and,
// for the residual stream, an fp32 copy; see core::Tensor::lo() / f32().
bool PreciseMode(int dt) { return dt == TTB_BF16 && core::PreciseBF16(); }

// out = LN(in) with the companion planes attached to `out` (already reshaped to its 16-bit shape). `in` is fp32 when
// in_f32, else of out's dtype.
void LayerNormPlanes(ttb_ctx* c, bool in_f32, const void* in, Tensor* out, const Tensor& gamma, const Tensor& beta, int64_t M, int64_t N,
                     float eps, bool want_f32, const char* name) {
  const int dt = core::ToTTBDtype(out->dtype());
  const auto shape = ShapeOf(*out);
  void* out_ptr = out->raw_mut();
  core::TensorExtras& ex = out->NewExtras();
  void* lo = ex.lo.Reshape(out->dtype(), shape, kDLCUDA, out->device_id(), "precise/lo_plane");
  float* f32 = want_f32 ? ex.f32.Reshape<float>(shape, kDLCUDA, out->device_id(), "precise/residual_stream") : nullptr;
  Check(ttb_layernorm_planes(c, in_f32 ? TTB_F32 : dt, dt, in, out_ptr, lo, f32, gamma.raw(), beta.raw(), M, N, eps), c, name);
}

// In-place layer norm of a 16-bit tensor that an int8 (per-row scheme) Linear produced: the int8 form of the result is
// written along and attached, because the next Linear of an int8 model will want it.
void LayerNormWithInt8(ttb_ctx* c, Tensor* t, const Tensor& gamma, const Tensor& beta, int64_t M, int64_t N, float eps, const char* name) {
  const int dt = core::ToTTBDtype(t->dtype());
  void* ptr = t->raw_mut();
  core::TensorExtras& ex = t->NewExtras();
  int8_t* q = static_cast<int8_t*>(ex.q8.Reshape(core::kInt8, {M, N}, kDLCUDA, t->device_id(), "linear/int8_activations"));
  float* s = ex.q8_scale.Reshape<float>({M}, kDLCUDA, t->device_id(), "linear/int8_row_scales");
  Check(ttb_layernorm_quant_int8(c, dt, ptr, ptr, q, s, gamma.raw(), beta.raw(), M, N, eps), c, name);
}

// dst (16-bit, [M, N]) = src (fp32): the re-layout kernel with an already K-major source is a plain conversion.
void CastFromF32(ttb_ctx* c, const float* src, int dst_dt, void* dst, int64_t M, int64_t N, const char* name) {
  Check(ttb_prepack_weight(c, TTB_F32, src, 1, N, M, dst_dt, dst), c, name);
}

// Which of the reference's two mask forms a tensor is (softmax.cpp:93-102): one row per batch or per query.
bool MaskIs2D(const Tensor& m) {
  return m.n_dim() == 2 || (m.n_dim() == 3 && m.shape(1) == 1) || (m.n_dim() == 4 && m.shape(2) == 1);
}

}  // namespace

// ===================================================================================================
// PackedLinear
// ===================================================================================================
const void* PackedLinear::Packed(bool is_trans) const {
  std::lock_guard<std::mutex> g(cache_->mu);
  Tensor& p = cache_->packed[is_trans ? 1 : 0];
  if (p.is_null()) {
    const int dt = FloatType(weight_, "linear weight");
    const int64_t K = in_dim(is_trans), N = out_dim(is_trans);
    ttb_ctx* c = DeviceContext(weight_.device_id());
    p.Reshape(weight_.dtype(), {N, K}, kDLCUDA, weight_.device_id(), "linear/packed_weight");
    Check(ttb_prepack_weight(c, dt, weight_.raw(), is_trans ? 1 : 0, K, N, dt, p.raw_mut()), c, "prepack_weight");
  }
  return p.raw();
}

const float* PackedLinear::PackedTf32(bool is_trans) const {
  std::lock_guard<std::mutex> g(cache_->mu);
  Tensor& p = cache_->tf32[is_trans ? 1 : 0];
  if (p.is_null()) {
    const int64_t K = in_dim(is_trans), N = out_dim(is_trans);
    ttb_ctx* c = DeviceContext(weight_.device_id());
    float* planes = p.Reshape<float>({2, N, K}, kDLCUDA, weight_.device_id(), "linear/tf32_weight_planes");
    Check(ttb_prepack_weight(c, TTB_F32, weight_.raw(), is_trans ? 1 : 0, K, N, TTB_F32, planes), c, "prepack_weight");
    Check(ttb_split_tf32(c, planes, N * K, planes, planes + N * K), c, "split_tf32");
  }
  return p.data<float>();
}

const float* PackedLinear::BiasF32() const {
  if (bias_.is_null()) return nullptr;
  std::lock_guard<std::mutex> g(cache_->mu);
  Tensor& b = cache_->bias_f32;
  if (b.is_null()) {
    // a [K=N, N=1] "weight" re-laid out is a plain dtype conversion of the vector
    const int dt = FloatType(bias_, "linear bias");
    ttb_ctx* c = DeviceContext(bias_.device_id());
    float* dst = b.Reshape<float>({bias_.numel()}, kDLCUDA, bias_.device_id(), "linear/bias_f32");
    Check(ttb_prepack_weight(c, dt, bias_.raw(), 1, bias_.numel(), 1, TTB_F32, dst), c, "bias to fp32");
  }
  return b.data<float>();
}

void PackedLinear::Int8(bool is_trans, const int8_t** wq, const float** scale, const int32_t** col_sum) const {
  std::lock_guard<std::mutex> g(cache_->mu);
  const int i = is_trans ? 1 : 0;
  if (col_sum) {  // the reference recipe's quantiser
    if (cache_->qref[i].is_null()) {
      const int dt = FloatType(weight_, "linear weight");
      const int64_t K = in_dim(is_trans), N = out_dim(is_trans);
      ttb_ctx* c = DeviceContext(weight_.device_id());
      cache_->qref[i].Reshape(core::kInt8, {N, K}, kDLCUDA, weight_.device_id(), "linear/int8_weight");
      cache_->qref_scale[i].Reshape(core::kFloat32, {1}, kDLCUDA, weight_.device_id(), "linear/int8_scale");
      cache_->qref_colsum[i].Reshape(core::kInt32, {N}, kDLCUDA, weight_.device_id(), "linear/int8_col_sum");
      Check(ttb_prepack_weight_int8_affine(c, dt, weight_.raw(), i, K, N, cache_->qref[i].mutableData<int8_t>(),
                                           cache_->qref_scale[i].mutableData<float>(), cache_->qref_colsum[i].mutableData<int32_t>()),
            c, "prepack_weight_int8_affine");
    }
    *wq = cache_->qref[i].data<int8_t>();
    *scale = cache_->qref_scale[i].data<float>();
    *col_sum = cache_->qref_colsum[i].data<int32_t>();
    return;
  }
  if (cache_->q[i].is_null()) {
    const int dt = FloatType(weight_, "linear weight");
    const int64_t K = in_dim(is_trans), N = out_dim(is_trans);
    ttb_ctx* c = DeviceContext(weight_.device_id());
    cache_->q[i].Reshape(core::kInt8, {N, K}, kDLCUDA, weight_.device_id(), "linear/int8_weight");
    cache_->qscale[i].Reshape(core::kFloat32, {1}, kDLCUDA, weight_.device_id(), "linear/int8_scale");
    Check(ttb_prepack_weight_int8(c, dt, weight_.raw(), i, K, N, cache_->q[i].mutableData<int8_t>(),
                                  cache_->qscale[i].mutableData<float>()),
          c, "prepack_weight_int8");
  }
  *wq = cache_->q[i].data<int8_t>();
  *scale = cache_->qscale[i].data<float>();
}

void PackedLinear::ForwardLayerNorm(const Tensor& x, int64_t M, const void* residual, const Tensor& gamma, const Tensor& beta, float eps,
                                    void* out, bool is_trans, const char* name) const {
  const int dt = FloatType(x, name);
  ttb_ctx* c = DeviceContext(x.device_id());
  const int64_t K = in_dim(is_trans), N = out_dim(is_trans);
  const bool two_planes = dt == TTB_BF16 && x.lo() && core::PreciseBF16();
  if (dt == TTB_F32 || use_int8() || bias_.is_null() || two_planes) {  // not the plain 16-bit product: two kernels
    Forward(x, M, TTB_EPI_BIAS_RESIDUAL, residual, out, is_trans, name);
    Check(ttb_layernorm(c, dt, out, out, gamma.raw(), beta.raw(), M, N, eps), c, name);
    return;
  }
  SameTypeDevice(x, weight_, name);
  TT_ENFORCE_EQ(x.shape(-1), K, "%s: input width %lld does not match the weight's %lld", name, (long long)x.shape(-1), (long long)K);
  Check(ttb_linear_layernorm(c, dt, x.raw(), K, Packed(is_trans), bias_.raw(), residual, N, gamma.raw(), beta.raw(), eps, M, N, K, out, N), c, name);
}

void PackedLinear::Forward(const Tensor& x, int64_t M, int epilogue, const void* residual, void* out, bool is_trans,
                           const char* name, int64_t ldo, void* out_lo, bool f32_out, Tensor* q8_of_out) const {
  const int dt = FloatType(x, name);
  SameTypeDevice(x, weight_, name);
  const int64_t K = in_dim(is_trans), N = out_dim(is_trans);
  TT_ENFORCE_EQ(x.shape(-1), K, "%s: input width %lld does not match the weight's %lld", name, (long long)x.shape(-1), (long long)K);
  ttb_ctx* c = DeviceContext(x.device_id());
  const void* bias = bias_.is_null() ? nullptr : bias_.raw();
  if (!bias && epilogue == TTB_EPI_BIAS) epilogue = TTB_EPI_NONE;
  if (ldo == 0) ldo = N;
  TT_ENFORCE(ldo == N || (dt != TTB_F32 && !use_int8()), "%s: a padded output pitch is only supported on the 16-bit path", name);
  TT_ENFORCE((!out_lo && !f32_out) || (dt == TTB_BF16 && !use_int8()), "%s: two-plane and fp32 outputs belong to the bf16 path", name);
  if (dt == TTB_F32 && core::Fp32TensorCores() && K % 4 == 0 && M > 0) {
    // fp32 on the tensor cores: activations split into two tf32 planes, weights kept as two planes, three products
    // accumulated in one GEMM with the elementwise kernel that followed MatMul in the reference as its epilogue
    // (mat_mul.cpp:81-96 selects tensor-op math for the same product)
    Tensor planes(nullptr);
    float* a = planes.Reshape<float>({2, M, K}, kDLCUDA, x.device_id(), "linear/tf32_activation_planes");
    Check(ttb_split_tf32(c, x.data<float>(), M * K, a, a + M * K), c, name);
    const float* w = PackedTf32(is_trans);
    ttb_linear_args args{};
    args.dtype = TTB_F32; args.out_dtype = TTB_F32;
    args.A = a; args.A2 = a + M * K; args.lda = K;
    args.W = w; args.W2 = w + N * K;
    args.bias = bias; args.residual = residual; args.ldr = N;
    args.M = M; args.N = N; args.K = K; args.epilogue = epilogue;
    args.out = out; args.ldo = N;
    Check(ttb_linear_ex(c, &args), c, name);
    return;
  }
  if (dt == TTB_F32) {
    // exact path: the reference's sequence MatMul -> elementwise kernel
    Check(ttb_matmul(c, dt, x.raw(), 0, weight_.raw(), is_trans ? 1 : 0, M, N, K, 1.0f, 0.0f, out), c, name);
    switch (epilogue) {
      case TTB_EPI_NONE: break;
      case TTB_EPI_BIAS: Check(ttb_add_bias(c, dt, out, bias, M, N), c, name); break;
      case TTB_EPI_BIAS_GELU: Check(ttb_add_bias_act(c, dt, out, bias, M, N, TTB_ACT_GELU), c, name); break;
      case TTB_EPI_BIAS_TANH: Check(ttb_add_bias_act(c, dt, out, bias, M, N, TTB_ACT_TANH), c, name); break;
      case TTB_EPI_BIAS_RESIDUAL: Check(ttb_add_input_bias(c, dt, out, residual, bias, M, N, out), c, name); break;
      default: TT_THROW("%s: unknown epilogue %d", name, epilogue);
    }
    return;
  }
  if (int8_mode_ == kInt8Reference) {
    const int8_t* wq;
    const float* ws;
    const int32_t* cs;
    Int8(is_trans, &wq, &ws, &cs);
    Tensor xq(nullptr), qp(nullptr);
    xq.Reshape(core::kInt8, {M, K}, kDLCUDA, x.device_id(), "linear/int8_activations");
    qp.Reshape(core::kFloat32, {4}, kDLCUDA, x.device_id(), "linear/int8_qparams");
    Check(ttb_quantize_tensor_affine(c, dt, x.raw(), M, K, xq.mutableData<int8_t>(), qp.mutableData<float>()), c, name);
    Check(ttb_linear_int8_affine(c, dt, xq.data<int8_t>(), qp.data<float>(), wq, ws, cs, bias, residual, N, M, N, K, epilogue, out, N), c, name);
    return;
  }
  if (use_int8()) {
    const int8_t* wq;
    const float* ws;
    Int8(is_trans, &wq, &ws);
    // The product; when the caller wants the int8 form of the output too (the next Linear is an int8 one), the epilogue
    // gathers the row maxima and one streaming pass quantises, instead of a quantiser that reads the output twice.
    auto product = [&](const int8_t* aq, const float* as) {
      static const bool fused_off = [] { const char* e = getenv("TTB_INT8_ROWMAX"); return e && e[0] == '0'; }();  // measurement switch
      // (below about a thousand rows the extra launches cost more than the second read they save)
      if (!q8_of_out || fused_off || N % 8 != 0 || N > 4096 || M < 1024) {
        Check(ttb_linear_int8(c, dt, aq, as, wq, ws, bias, residual, N, M, N, K, epilogue, out, N), c, name);
        return;
      }
      Tensor maxima(nullptr);
      float* am = maxima.Reshape<float>({M}, kDLCUDA, x.device_id(), "linear/int8_row_maxima");
      Check(ttb_linear_int8_rowmax(c, dt, aq, as, wq, ws, bias, residual, N, M, N, K, epilogue, out, N, am), c, name);
      core::TensorExtras& ex = q8_of_out->NewExtras();
      int8_t* q = static_cast<int8_t*>(ex.q8.Reshape(core::kInt8, {M, N}, kDLCUDA, x.device_id(), "linear/int8_activations"));
      float* qs = ex.q8_scale.Reshape<float>({M}, kDLCUDA, x.device_id(), "linear/int8_row_scales");
      Check(ttb_quantize_rows_int8_given_max(c, dt, out, M, N, am, q, qs), c, name);
    };
    if (x.q8() && x.q8_scale() && x.q8()->numel() == M * K) {  // the producer already quantised this activation
      product(x.q8()->data<int8_t>(), x.q8_scale()->data<float>());
      return;
    }
    Tensor xq(nullptr), xs(nullptr);
    xq.Reshape(core::kInt8, {M, K}, kDLCUDA, x.device_id(), "linear/int8_activations");
    xs.Reshape(core::kFloat32, {M}, kDLCUDA, x.device_id(), "linear/int8_row_scales");
    Check(ttb_quantize_rows_int8(c, dt, x.raw(), M, K, xq.mutableData<int8_t>(), xs.mutableData<float>()), c, name);
    product(xq.data<int8_t>(), xs.data<float>());
    return;
  }
  if (ldo != N) epilogue |= TTB_EPI_FLAG_ROW_PADDING_IS_SCRATCH;  // only Linear's own row-padded scratch gets here
  ttb_linear_args args{};
  args.dtype = dt; args.out_dtype = f32_out ? TTB_F32 : dt;
  args.A = x.raw(); args.lda = K;
  // a bf16 activation that carries what its rounding dropped is used whole: A . W + A_lo . W
  if (dt == TTB_BF16 && x.lo() && core::PreciseBF16()) args.A2 = x.lo()->raw();
  args.W = Packed(is_trans);
  args.bias = f32_out ? static_cast<const void*>(BiasF32()) : bias;
  args.residual = residual; args.ldr = N;
  args.M = M; args.N = N; args.K = K; args.epilogue = epilogue;
  args.out = out; args.out_lo = out_lo; args.ldo = ldo;
  Check(ttb_linear_ex(c, &args), c, name);
}

// ===================================================================================================
// BERTEmbedding
// ===================================================================================================
void BERTEmbedding::EnforceShapeAndType() const {
  TT_ENFORCE_EQ(word_embedings_.n_dim(), 2, "word embeddings must be a matrix");
  TT_ENFORCE_EQ(position_embeddings_.n_dim(), 2, "position embeddings must be a matrix");
  TT_ENFORCE_EQ(token_type_embeddings_.n_dim(), 2, "token type embeddings must be a matrix");
  TT_ENFORCE_EQ(word_embedings_.shape(1), position_embeddings_.shape(1), "embedding widths differ");
  TT_ENFORCE_EQ(word_embedings_.shape(1), layer_norm_weights_.shape(0), "layer norm width differs from the embedding width");
}

void BERTEmbedding::operator()(const Tensor& input_ids, const Tensor& position_ids, const Tensor& token_type_ids,
                               Tensor* output_tensor) const {
  TT_ENFORCE_EQ(input_ids.n_dim(), 2, "The input ids should be a matrix with shape [BatchSize, SeqLen].");
  TT_ENFORCE(output_tensor, "The output tensor should not be nullptr.");
  const int dt = FloatType(word_embedings_, "word embeddings");
  TT_ENFORCE(input_ids.on_gpu(), "input ids must be on the GPU");
  const int64_t B = input_ids.shape(0), L = input_ids.shape(1), H = word_embedings_.shape(1);
  const int dev = input_ids.device_id();
  ttb_ctx* c = DeviceContext(dev);
  output_tensor->Reshape(word_embedings_.dtype(), {B, L, H}, kDLCUDA, dev, "BERTEmbedding/Reshape");
  void* out = output_tensor->raw_mut();
  void* lo = nullptr;
  float* f32 = nullptr;
  if (PreciseMode(dt)) {
    core::TensorExtras& ex = output_tensor->NewExtras();
    lo = ex.lo.Reshape(word_embedings_.dtype(), {B, L, H}, kDLCUDA, dev, "precise/lo_plane");
    f32 = ex.f32.Reshape<float>({B, L, H}, kDLCUDA, dev, "precise/residual_stream");
  }
  Check(ttb_embedding_ln_planes(c, dt, input_ids.data<int64_t>(), position_ids.is_null() ? nullptr : position_ids.data<int64_t>(),
                                token_type_ids.is_null() ? nullptr : token_type_ids.data<int64_t>(), nullptr, B, L, B * L,
                                word_embedings_.raw(), position_embeddings_.raw(), token_type_embeddings_.raw(),
                                layer_norm_weights_.raw(), layer_norm_bias_.raw(), H, word_embedings_.shape(0),
                                position_embeddings_.shape(0), token_type_embeddings_.shape(0), 1e-12f, out, lo, f32),
        c, "BERTEmbedding");
}

void BERTEmbedding::Packed(const Tensor& input_ids, const std::vector<int64_t>& seq_lens, Tensor* output_tensor,
                           const Tensor& position_ids, const Tensor& token_type_ids) const {
  const int dt = FloatType(word_embedings_, "word embeddings");
  TT_ENFORCE(input_ids.on_gpu(), "input ids must be on the GPU");
  const int64_t T = input_ids.numel(), H = word_embedings_.shape(1);
  TT_ENFORCE_EQ(T, std::accumulate(seq_lens.begin(), seq_lens.end(), (int64_t)0), "ids do not match the sequence lengths");
  TT_ENFORCE(position_ids.is_null() || (position_ids.on_gpu() && position_ids.numel() == T), "packed position ids must be %lld ids on the GPU", (long long)T);
  TT_ENFORCE(token_type_ids.is_null() || (token_type_ids.on_gpu() && token_type_ids.numel() == T), "packed token type ids must be %lld ids on the GPU", (long long)T);
  const int dev = input_ids.device_id();
  ttb_ctx* c = DeviceContext(dev);
  output_tensor->Reshape(word_embedings_.dtype(), {1, T, H}, kDLCUDA, dev, "BERTEmbedding/Reshape");
  void* out = output_tensor->raw_mut();
  void* lo = nullptr;
  float* f32 = nullptr;
  if (PreciseMode(dt)) {
    core::TensorExtras& ex = output_tensor->NewExtras();
    lo = ex.lo.Reshape(word_embedings_.dtype(), {1, T, H}, kDLCUDA, dev, "precise/lo_plane");
    f32 = ex.f32.Reshape<float>({1, T, H}, kDLCUDA, dev, "precise/residual_stream");
  }
  const core::CuSeqlensHandle cu = core::CuSeqlens(dev, seq_lens);
  Check(ttb_embedding_ln_planes(c, dt, input_ids.data<int64_t>(), position_ids.is_null() ? nullptr : position_ids.data<int64_t>(),
                                token_type_ids.is_null() ? nullptr : token_type_ids.data<int64_t>(), cu.get(), (int64_t)seq_lens.size(), 0, T,
                                word_embedings_.raw(), position_embeddings_.raw(), token_type_embeddings_.raw(), layer_norm_weights_.raw(),
                                layer_norm_bias_.raw(), H, word_embedings_.shape(0), position_embeddings_.shape(0),
                                token_type_embeddings_.shape(0), 1e-12f, out, lo, f32),
        c, "BERTEmbedding/packed");
}

// ===================================================================================================
// MultiHeadedAttention
// ===================================================================================================
MultiHeadedAttention::MultiHeadedAttention(Tensor k_weight, Tensor k_bias, Tensor v_weight, Tensor v_bias, Tensor q_weight,
                                           Tensor q_bias, Tensor dense_weight, Tensor dense_bias, Tensor qkv_weight, Tensor qkv_bias,
                                           int64_t num_attention_heads)
    : k_(std::move(k_weight), std::move(k_bias)), v_(std::move(v_weight), std::move(v_bias)), q_(std::move(q_weight), std::move(q_bias)),
      qkv_(std::move(qkv_weight), std::move(qkv_bias)), dense_(std::move(dense_weight), std::move(dense_bias)),
      layernorm_gamma_(nullptr), layernorm_beta_(nullptr), num_attention_heads_(num_attention_heads) {
  EnforceShapeAndType();
}

MultiHeadedAttention::MultiHeadedAttention(Tensor k_weight, Tensor k_bias, Tensor v_weight, Tensor v_bias, Tensor q_weight,
                                           Tensor q_bias, Tensor dense_weight, Tensor dense_bias, Tensor qkv_weight, Tensor qkv_bias,
                                           Tensor layernorm_gamma, Tensor layernorm_beta, int64_t num_attention_heads)
    : k_(std::move(k_weight), std::move(k_bias)), v_(std::move(v_weight), std::move(v_bias)), q_(std::move(q_weight), std::move(q_bias)),
      qkv_(std::move(qkv_weight), std::move(qkv_bias)), dense_(std::move(dense_weight), std::move(dense_bias)),
      layernorm_gamma_(std::move(layernorm_gamma)), layernorm_beta_(std::move(layernorm_beta)),
      num_attention_heads_(num_attention_heads) {
  EnforceShapeAndType();
}

void MultiHeadedAttention::EnforceShapeAndType() const {
  const bool has_qkv = !qkv_.weight().is_null() && !qkv_.bias().is_null();
  const bool has_split = !q_.weight().is_null() && !k_.weight().is_null() && !v_.weight().is_null() && !q_.bias().is_null() &&
                         !k_.bias().is_null() && !v_.bias().is_null();
  TT_ENFORCE(has_qkv || has_split, "attention needs the fused qkv weight and bias (self) or separate q, k, v weights and biases (context)");
  if (has_qkv) TT_ENFORCE_EQ(qkv_.weight().n_dim(), 2, "qkv weight must be a matrix");
  TT_ENFORCE_EQ(dense_.weight().n_dim(), 2, "dense weight must be a matrix");
  TT_ENFORCE(num_attention_heads_ > 0, "number of heads must be positive");
}

void MultiHeadedAttention::operator()(const Tensor& key_tensor, const Tensor& value_tensor, const Tensor& query_tensor,
                                      const Tensor& attention_mask, const std::string& attn_type, Tensor* output,
                                      Tensor* att_score, std::unordered_map<std::string, Tensor*> layer_cache,
                                      bool pre_layernorm, bool post_layernorm, bool post_add_input, bool is_trans_weight) const {
  TT_ENFORCE_EQ(key_tensor.n_dim(), 3, "The key_tensor should be a matrix with shape [batch_size, key_seq_len, hidden_size].");
  TT_ENFORCE_EQ(value_tensor.n_dim(), 3, "The value_tensor should be a matrix with shape [batch_size, key_seq_len, hidden_size].");
  TT_ENFORCE_EQ(query_tensor.n_dim(), 3, "The query_tensors should be a matrix with shape [batch_size, query_seq_len, hidden_size].");
  if (attn_type == "context") {
    // layer_cache["memory_keys" / "memory_values"]: absent = nothing is kept; present and null = computed by this call and
    // kept; present and filled = used instead of projecting key_tensor / value_tensor again.
    Tensor *mem_k = nullptr, *mem_v = nullptr;
    for (auto& kv : layer_cache) {
      if (kv.first == "memory_keys") mem_k = kv.second;
      else if (kv.first == "memory_values") mem_v = kv.second;
    }
    TT_ENFORCE((mem_k == nullptr) == (mem_v == nullptr), "layer_cache needs both memory_keys and memory_values");
    RunContext(key_tensor, value_tensor, query_tensor, attention_mask, output, att_score, mem_k, mem_v, pre_layernorm, post_layernorm,
               post_add_input, is_trans_weight);
    return;
  }
  if (attn_type != "self") TT_THROW("attn_type should be context or self.");
  // Incremental decoding (multi_headed_attention.cpp:207-231): the reference concatenates the step's keys / values to
  // layer_cache["self_keys" / "self_values"] ([B, heads, T, d] there). Here the two entries are appended in place: their shape
  // reads [T, B, H] (T = tokens cached), their buffer is paged and opaque to the caller; an entry that is present but still
  // empty starts the cache.
  Tensor *cache_k = nullptr, *cache_v = nullptr;
  for (auto& kv : layer_cache) {
    if (kv.first == "self_keys") cache_k = kv.second;
    else if (kv.first == "self_values") cache_v = kv.second;
  }
  TT_ENFORCE((cache_k == nullptr) == (cache_v == nullptr), "layer_cache needs both self_keys and self_values");
  Run(query_tensor, attention_mask, nullptr, output, att_score, pre_layernorm, post_layernorm, post_add_input, is_trans_weight, cache_k,
      cache_v);
}

namespace {
// Makes a cache hold past + n_new tokens, keeping the first `past`. The tensor's shape is the logical [T, B, H]; its buffer is
// paged ([pages, B, 16, H], see ttb_attention_decode) and reserved ahead (a Tensor keeps its buffer across Reshape calls while
// it is large enough), so most steps only change the logical shape; when the reserve runs out the pages move to a buffer
// twice as long.
void EnsureCacheRows(Tensor* t, DLDataType dtype, int64_t past, int64_t n_new, int64_t B, int64_t H, int dev) {
  const std::vector<int64_t> want{past + n_new, B, H};
  auto pages = [](int64_t tokens) { return (tokens + 15) / 16; };
  const size_t need = (size_t)(pages(past + n_new) * 16 * B * H) * 2;
  if (past == 0) {
    t->Reshape(dtype, {16 * pages(std::max<int64_t>(2 * n_new, n_new + 256)), B, H}, kDLCUDA, dev, "layer_cache/reserve");
  } else if (t->capacity_bytes() < need) {
    ttb_ctx* c = DeviceContext(dev);
    Tensor bigger(nullptr);
    bigger.Reshape(dtype, {16 * pages(2 * (past + n_new)), B, H}, kDLCUDA, dev, "layer_cache/grow");
    const size_t old_bytes = (size_t)(pages(past) * 16 * B * H) * 2;
    Check(ttb_copy_2d(c, bigger.raw_mut(), old_bytes, t->raw(), old_bytes, old_bytes, 1), c, "layer_cache/grow");
    Check(ttb_ctx_sync(c), c, "layer_cache/grow");  // the old buffer is released when `*t` is overwritten
    *t = std::move(bigger);
  }
  t->Reshape(dtype, want, kDLCUDA, dev, "layer_cache");
}
}  // namespace

void MultiHeadedAttentionSmartBatch::operator()(const Tensor& key_tensor, const Tensor& value_tensor, const Tensor& query_tensor,
                                                const Tensor& attention_mask, const std::string& attn_type, Tensor* output,
                                                Tensor* att_score, std::unordered_map<std::string, Tensor*> layer_cache,
                                                const std::vector<int64_t>& query_seq_len_list,
                                                const std::vector<int64_t>& key_seq_len_list, bool pre_layernorm,
                                                bool post_layernorm, bool post_add_input, bool is_trans_weight) const {
  TT_ENFORCE_EQ(query_tensor.n_dim(), 3, "The query_tensors should be a matrix with shape [1, sum_query_seq_len, hidden_size].");
  TT_ENFORCE_EQ(query_tensor.shape(0), 1, "The packed query tensor's first dimension must be 1.");
  TT_ENFORCE(!query_seq_len_list.empty(), "query_seq_len_list is empty");
  const int64_t total = std::accumulate(query_seq_len_list.begin(), query_seq_len_list.end(), (int64_t)0);
  TT_ENFORCE_EQ(query_tensor.shape(1), total, "The query_tensor shape 1 should be the sum of seq_len_list.");
  if (attn_type == "context") {
    // multi_headed_attention_smart_batch.cpp:34-170: queries of one set of lengths against keys / values of another
    TT_ENFORCE_EQ(key_seq_len_list.size(), query_seq_len_list.size(), "query_seq_len_list and key_seq_len_list differ in batch size");
    Tensor *mem_k = nullptr, *mem_v = nullptr;
    for (auto& kv : layer_cache) {
      if (kv.first == "memory_keys") mem_k = kv.second;
      else if (kv.first == "memory_values") mem_v = kv.second;
    }
    TT_ENFORCE((mem_k == nullptr) == (mem_v == nullptr), "layer_cache needs both memory_keys and memory_values");
    RunContext(key_tensor, value_tensor, query_tensor, attention_mask, output, att_score, mem_k, mem_v, pre_layernorm, post_layernorm,
               post_add_input, is_trans_weight, &query_seq_len_list, &key_seq_len_list);
    return;
  }
  if (attn_type != "self") TT_THROW("attn_type should be context or self.");
  for (auto& kv : layer_cache)
    if (kv.second && !kv.second->is_null())
      TT_THROW("the packed self-attention takes no key/value cache (decode with the fixed-length MultiHeadedAttention)");
  Run(query_tensor, attention_mask, &query_seq_len_list, output, att_score, pre_layernorm, post_layernorm, post_add_input,
      is_trans_weight);
}

void BertAttention::operator()(const Tensor& input_tensor, const Tensor& attention_mask, Tensor* output, Tensor* attn,
                               bool is_trans_weight) const {
  // bert_attention.cpp:29-47 of the reference: self attention with post layer norm
  TT_ENFORCE_EQ(input_tensor.n_dim(), 3, "The input should be [batch_size, seq_len, hidden_size].");
  Run(input_tensor, attention_mask, nullptr, output, attn, false, true, false, is_trans_weight);
}

void MultiHeadedAttention::Run(const Tensor& x, const Tensor& attention_mask, const std::vector<int64_t>* seq_lens, Tensor* output,
                               Tensor* att_score, bool pre_layernorm, bool post_layernorm, bool post_add_input,
                               bool is_trans_weight, Tensor* cache_keys, Tensor* cache_values) const {
  TT_ENFORCE(output, "The output tensor should not be nullptr.");
  TT_ENFORCE(!qkv_.weight().is_null(), "self attention needs the fused qkv weight and bias");
  const int dt = FloatType(x, "attention input");
  SameTypeDevice(x, qkv_.weight(), "attention");
  const int dev = x.device_id();
  ttb_ctx* c = DeviceContext(dev);
  const int64_t H = x.shape(2), heads = num_attention_heads_, d = H / heads;
  TT_ENFORCE_EQ(d * heads, H, "hidden size %lld is not divisible by %lld heads", (long long)H, (long long)heads);
  TT_ENFORCE_EQ(qkv_.out_dim(is_trans_weight), 3 * H, "qkv weight does not map hidden -> 3*hidden");
  const int64_t B = seq_lens ? (int64_t)seq_lens->size() : x.shape(0);
  const int64_t T = seq_lens ? x.shape(1) : x.shape(0) * x.shape(1);
  const int64_t maxL = seq_lens ? *std::max_element(seq_lens->begin(), seq_lens->end()) : x.shape(1);
  if (pre_layernorm || post_layernorm) TT_ENFORCE(!layernorm_gamma_.is_null(), "this attention layer was built without layer norm weights");
  const float scale = 1.0f / std::sqrt((float)d);
  const auto out_shape = ShapeOf(x);

  // 1) optional pre layer norm into a temporary (the input itself is the residual)
  Tensor normed(nullptr);
  const Tensor* gemm_in = &x;
  if (pre_layernorm) {
    normed.Reshape(x.dtype(), out_shape, kDLCUDA, dev, "self/layernorm/Reshape");
    if (PreciseMode(dt)) {
      LayerNormPlanes(c, x.f32() != nullptr, x.f32() ? x.f32()->raw() : x.raw(), &normed, layernorm_gamma_, layernorm_beta_, T, H, pre_ln_eps_,
                      false, "self/layernorm");
    } else {
      Check(ttb_layernorm(c, dt, x.raw(), normed.raw_mut(), layernorm_gamma_.raw(), layernorm_beta_.raw(), T, H, pre_ln_eps_), c,
            "self/layernorm");
    }
    gemm_in = &normed;
  }

  const bool fused = dt != TTB_F32 && att_score == nullptr && d == 64;
  Tensor context(nullptr);  // [T, H] token-major attention output
  context.Reshape(x.dtype(), {T, H}, kDLCUDA, dev, "batch_gemm4/Reshape");

  if (fused) {
    // 2) QKV projection with the bias in the GEMM epilogue, left token-major [T, 3H]
    Tensor qkv(nullptr);
    qkv.Reshape(x.dtype(), {T, 3 * H}, kDLCUDA, dev, "self/qkv_out1/Reshape");
    qkv_.Forward(*gemm_in, T, TTB_EPI_BIAS, nullptr, qkv.raw_mut(), is_trans_weight, "self/gemm012_fused");
    // 3) attention over packed tokens; the mask tensor (if any) is applied as the reference does
    const core::CuSeqlensHandle cu_handle = seq_lens ? core::CuSeqlens(dev, *seq_lens) : core::UniformCuSeqlens(dev, B, maxL);
    const int32_t* cu = cu_handle.get();
    const float* mask = nullptr;
    int64_t mbs = 0, mrs = 0;
    if (!attention_mask.is_null()) {
      TT_ENFORCE(attention_mask.on_gpu() && core::SameType(attention_mask.dtype(), core::kFloat32),
                 "the attention mask must be an fp32 tensor on the GPU");
      mask = attention_mask.data<float>();
      const int64_t Lk = attention_mask.shape(-1);
      TT_ENFORCE_GE(Lk, maxL, "attention mask is shorter than the longest sequence");
      if (MaskIs2D(attention_mask)) { mbs = Lk; mrs = 0; }
      else { mrs = Lk; mbs = attention_mask.shape(-2) * Lk; }
    }
    if (cache_keys) {
      TT_ENFORCE(!seq_lens && !mask, "layer_cache decoding takes equal-length batches without a mask tensor");
      const int64_t past = cache_keys->is_null() ? 0 : cache_keys->shape(0);
      TT_ENFORCE(cache_values->is_null() ? past == 0 : cache_values->shape(0) == past, "self_keys and self_values disagree on the cached length");
      if (past > 0) {
        TT_ENFORCE(cache_keys->shape(1) == B && cache_keys->shape(2) == H && core::SameType(cache_keys->dtype(), x.dtype()),
                   "layer_cache does not match this batch ([T, %lld, %lld] expected)", (long long)B, (long long)H);
      }
      EnsureCacheRows(cache_keys, x.dtype(), past, maxL, B, H, dev);
      EnsureCacheRows(cache_values, x.dtype(), past, maxL, B, H, dev);
      if (past == 0) {  // prompt: regular attention over the new tokens, then file their keys / values
        Check(ttb_attention_fwd(c, dt, qkv.raw(), T, cu, B, maxL, heads, d, nullptr, 0, 0, causal_ ? 1 : 0, scale, context.raw_mut()), c,
              "attention_fwd");
        Check(ttb_kv_cache_append(c, dt, qkv.raw(), B, maxL, heads, d, cache_keys->raw_mut(), cache_values->raw_mut(), 0), c, "kv_cache_append");
      } else {
        Check(ttb_attention_decode(c, dt, qkv.raw(), B, maxL, heads, d, cache_keys->raw_mut(), cache_values->raw_mut(), past, scale,
                                   context.raw_mut()),
              c, "attention_decode");
      }
    } else {
      Check(ttb_attention_fwd(c, dt, qkv.raw(), T, cu, B, maxL, heads, d, mask, mbs, mrs, causal_ ? 1 : 0, scale, context.raw_mut()), c,
            "attention_fwd");
    }
    if (att_score) *att_score = Tensor(nullptr);
  } else {
    // The reference's own sequence (multi_headed_attention.cpp:168-232,320-354), scores materialised.
    TT_ENFORCE(!cache_keys, "layer_cache decoding is provided for 16-bit models with 64-wide heads");
    TT_ENFORCE(!causal_ || !attention_mask.is_null(), "the unfused path needs an explicit mask tensor for causal attention");
    Tensor qkv(nullptr), q(nullptr), k(nullptr), v(nullptr), ctx_heads(nullptr), scores_local(nullptr);
    qkv.Reshape(x.dtype(), {T, 3 * H}, kDLCUDA, dev, "self/qkv_out1/Reshape");
    qkv_.Forward(*gemm_in, T, TTB_EPI_NONE, nullptr, qkv.raw_mut(), is_trans_weight, "self/gemm012_fused");
    const std::vector<int64_t> head_shape{B, heads, maxL, d};
    q.Reshape(x.dtype(), head_shape, kDLCUDA, dev, "self/q/Reshape");
    k.Reshape(x.dtype(), head_shape, kDLCUDA, dev, "self/k/Reshape");
    v.Reshape(x.dtype(), head_shape, kDLCUDA, dev, "self/v/Reshape");
    const core::CuSeqlensHandle cu_handle = seq_lens ? core::CuSeqlens(dev, *seq_lens) : core::CuSeqlensHandle();
    const int32_t* cu = cu_handle.get();
    Check(ttb_split_add_bias_transpose_pad(c, dt, qkv.raw(), qkv_.bias().raw(), cu, B, maxL, heads, d, q.raw_mut(), k.raw_mut(),
                                           v.raw_mut()),
          c, "self/SplitAddBiasTransposeForScore");
    Tensor* scores = att_score ? att_score : &scores_local;
    scores->Reshape(x.dtype(), {B, heads, maxL, maxL}, kDLCUDA, dev, "batch_gemm3/Reshape");
    Check(ttb_batch_matmul(c, dt, q.raw(), 0, k.raw(), 1, B * heads, maxL, maxL, d, scale, 0.0f, scores->raw_mut()), c, "batch_gemm3");
    const float* mask = nullptr;
    int is2d = 1;
    Tensor pad_mask(nullptr);
    if (attention_mask.is_null() && seq_lens) {
      // Packed input without a mask tensor: keys beyond each sequence's length are padding. Build the
      // [B,1,maxL] additive mask the reference's Python layer builds (modeling_smart_pad.py:82-98).
      std::vector<float> host_mask((size_t)(B * maxL), 0.f);
      for (int64_t b = 0; b < B; ++b)
        for (int64_t l = (*seq_lens)[b]; l < maxL; ++l) host_mask[b * maxL + l] = -1e9f;
      float* dm = pad_mask.Reshape<float>({B, 1, maxL}, kDLCUDA, dev, "self/pad_mask");
      Check(ttb_memcpy_h2d(c, dm, host_mask.data(), host_mask.size() * sizeof(float)), c, "self/pad_mask");
      mask = dm;
    }
    if (!attention_mask.is_null()) {
      TT_ENFORCE(attention_mask.on_gpu() && core::SameType(attention_mask.dtype(), core::kFloat32),
                 "the attention mask must be an fp32 tensor on the GPU");
      TT_ENFORCE_EQ(attention_mask.shape(-1), maxL, "attention mask width must equal the (padded) key length");
      mask = attention_mask.data<float>();
      is2d = MaskIs2D(attention_mask) ? 1 : 0;
    }
    Check(ttb_mask_softmax(c, dt, scores->raw_mut(), mask, B, heads, maxL, maxL, 1.0f, is2d), c, "ApplyMaskAndSoftmax");
    ctx_heads.Reshape(x.dtype(), head_shape, kDLCUDA, dev, "ApplyMaskAndSoftmax/Reshape");
    Check(ttb_batch_matmul(c, dt, scores->raw(), 0, v.raw(), 0, B * heads, maxL, d, maxL, 1.0f, 0.0f, ctx_heads.raw_mut()), c,
          "batch_gemm4");
    Check(ttb_transpose_for_score_pad(c, dt, ctx_heads.raw(), cu, B, maxL, heads, d, context.raw_mut()), c, "TransposeForScore");
  }

  // 4) output projection and what follows it
  Finish(context, x, T, output, post_layernorm, post_add_input, is_trans_weight);
}

void MultiHeadedAttention::Finish(const Tensor& context, const Tensor& x, int64_t T, Tensor* output, bool post_layernorm,
                                  bool post_add_input, bool is_trans_weight) const {
  const int dt = FloatType(x, "attention input");
  const int dev = x.device_id();
  ttb_ctx* c = DeviceContext(dev);
  const int64_t H = x.shape(2);
  output->Reshape(x.dtype(), ShapeOf(x), kDLCUDA, dev, "gemm5/Reshape");
  const bool precise = PreciseMode(dt) && x.f32() != nullptr && !dense_.use_int8();
  if (precise && (post_add_input || post_layernorm)) {
    // the residual stream stays fp32: out-projection + bias + fp32 residual -> fp32, then either the layer norm that
    // writes the next GEMM's two operand planes, or (pre-LN models) the 16-bit copy the caller sees
    if (post_layernorm) {
      Tensor sum(nullptr);
      float* s = sum.Reshape<float>(ShapeOf(x), kDLCUDA, dev, "gemm5/fp32_sum");
      dense_.Forward(context, T, TTB_EPI_BIAS_RESIDUAL, x.f32()->raw(), s, is_trans_weight, "gemm5", 0, nullptr, true);
      LayerNormPlanes(c, true, s, output, layernorm_gamma_, layernorm_beta_, T, H, 1e-12f, true, "AddBiasLayerNorm");
    } else {
      void* pub = output->raw_mut();
      core::TensorExtras& ex = output->NewExtras();
      float* s = ex.f32.Reshape<float>(ShapeOf(x), kDLCUDA, dev, "precise/residual_stream");
      dense_.Forward(context, T, TTB_EPI_BIAS_RESIDUAL, x.f32()->raw(), s, is_trans_weight, "gemm5", 0, nullptr, true);
      CastFromF32(c, s, dt, pub, T, H, "gemm5/public_copy");
    }
    return;
  }
  if (post_add_input) {
    dense_.Forward(context, T, TTB_EPI_BIAS_RESIDUAL, x.raw(), output->raw_mut(), is_trans_weight, "gemm5");
  } else if (!post_layernorm) {
    dense_.Forward(context, T, TTB_EPI_BIAS, nullptr, output->raw_mut(), is_trans_weight, "gemm5");
  } else if (dt == TTB_F32) {
    dense_.Forward(context, T, TTB_EPI_NONE, nullptr, output->raw_mut(), is_trans_weight, "gemm5");
    Check(ttb_add_bias_layernorm(c, dt, output->raw_mut(), x.raw(), dense_.bias().raw(), layernorm_gamma_.raw(),
                                 layernorm_beta_.raw(), T, H, 1e-12f),
          c, "AddBiasLayerNorm");
  } else {
    if (dense_.int8_mode() == PackedLinear::kInt8PerRow) {
      dense_.Forward(context, T, TTB_EPI_BIAS_RESIDUAL, x.raw(), output->raw_mut(), is_trans_weight, "gemm5");
      LayerNormWithInt8(c, output, layernorm_gamma_, layernorm_beta_, T, H, 1e-12f, "AddBiasLayerNorm");
    } else {  // one kernel where the shape allows it: projection + bias + residual + layer norm
      dense_.ForwardLayerNorm(context, T, x.raw(), layernorm_gamma_, layernorm_beta_, 1e-12f, output->raw_mut(), is_trans_weight, "gemm5");
    }
  }
}

void MultiHeadedAttention::RunContext(const Tensor& key_tensor, const Tensor& value_tensor, const Tensor& query_tensor,
                                      const Tensor& attention_mask, Tensor* output, Tensor* att_score, Tensor* memory_keys,
                                      Tensor* memory_values, bool pre_layernorm, bool post_layernorm, bool post_add_input,
                                      bool is_trans_weight, const std::vector<int64_t>* q_lens,
                                      const std::vector<int64_t>* k_lens) const {
  // The reference's sequence (multi_headed_attention.cpp:45-167, 308-354) on this library's kernels: three separate
  // projections, AddBiasTransposeForScore into [B, heads, L, d], scores materialised, mask + softmax, weighted values,
  // transpose back, output projection. The encoder memory's keys / values are projected once per sequence when the caller
  // passes layer_cache entries, so a decoding step costs one query projection and two small batched products.
  TT_ENFORCE(output, "The output tensor should not be nullptr.");
  TT_ENFORCE(!q_.weight().is_null() && !k_.weight().is_null() && !v_.weight().is_null(),
             "context attention needs the separate q, k, v weights and biases");
  const Tensor& x = query_tensor;
  const int dt = FloatType(x, "attention input");
  SameTypeDevice(x, q_.weight(), "attention");
  const int dev = x.device_id();
  ttb_ctx* c = DeviceContext(dev);
  const bool packed = q_lens != nullptr;
  TT_ENFORCE(packed == (k_lens != nullptr), "packed context attention needs both length lists");
  const int64_t H = x.shape(2), heads = num_attention_heads_, d = H / heads;
  const int64_t B = packed ? (int64_t)q_lens->size() : x.shape(0);
  const int64_t Lq = packed ? *std::max_element(q_lens->begin(), q_lens->end()) : x.shape(1);  // padded query length
  const int64_t T = x.rows();
  // prefix sums of the packed rows (null handles = equal lengths, rows b * L + l)
  const core::CuSeqlensHandle cu_q = packed ? core::CuSeqlens(dev, *q_lens) : core::CuSeqlensHandle();
  const core::CuSeqlensHandle cu_k = packed ? core::CuSeqlens(dev, *k_lens) : core::CuSeqlensHandle();
  TT_ENFORCE_EQ(d * heads, H, "hidden size %lld is not divisible by %lld heads", (long long)H, (long long)heads);
  TT_ENFORCE_EQ(q_.out_dim(is_trans_weight), H, "q weight does not map hidden -> hidden");
  if (pre_layernorm || post_layernorm) TT_ENFORCE(!layernorm_gamma_.is_null(), "this attention layer was built without layer norm weights");
  const float scale = 1.0f / std::sqrt((float)d);

  // 1) queries
  Tensor normed(nullptr), lin(nullptr), q(nullptr);
  const Tensor* q_in = &x;
  if (pre_layernorm) {
    normed.Reshape(x.dtype(), ShapeOf(x), kDLCUDA, dev, "context/gemm0/q_out2/Reshape");
    Check(ttb_layernorm(c, dt, x.raw(), normed.raw_mut(), layernorm_gamma_.raw(), layernorm_beta_.raw(), T, H, pre_ln_eps_), c,
          "context/gemm0/prelayernorm");
    q_in = &normed;
  }
  lin.Reshape(x.dtype(), {T, H}, kDLCUDA, dev, "context/gemm0/q_out1/Reshape");
  q_.Forward(*q_in, T, TTB_EPI_NONE, nullptr, lin.raw_mut(), is_trans_weight, "context/gemm0");
  q.Reshape(x.dtype(), {B, heads, Lq, d}, kDLCUDA, dev, "context/AddBiasTransposeForScore/q_out2/Reshape");
  Check(ttb_add_bias_transpose_for_score_pad(c, dt, lin.raw(), q_.bias().raw(), cu_q.get(), B, Lq, heads, d, q.raw_mut()), c,
        "context/AddBiasTransposeForScore");

  // 2) keys / values: from the cache when it is filled, otherwise projected (and filed when a cache entry was passed)
  Tensor k_local(nullptr), v_local(nullptr);
  Tensor *k = &k_local, *v = &v_local;
  const bool memory_filled = memory_keys && !memory_keys->is_null() && !memory_values->is_null();
  if (memory_filled) {
    k = memory_keys;
    v = memory_values;
    TT_ENFORCE(k->n_dim() == 4 && k->shape(0) == B && k->shape(1) == heads && k->shape(3) == d && core::SameType(k->dtype(), x.dtype()),
               "layer_cache memory_keys does not match this batch ([%lld, %lld, Lk, %lld] expected)", (long long)B, (long long)heads, (long long)d);
    TT_ENFORCE(v->n_dim() == 4 && v->shape(0) == B && v->shape(1) == heads && v->shape(2) == k->shape(2) && v->shape(3) == d &&
                   core::SameType(v->dtype(), x.dtype()),
               "layer_cache memory_values does not match memory_keys");
  } else {
    if (packed) {
      const int64_t sum_k = std::accumulate(k_lens->begin(), k_lens->end(), (int64_t)0);
      TT_ENFORCE(key_tensor.shape(0) == 1 && key_tensor.shape(1) == sum_k, "The key_tensor shape 1 should be the sum of seq_len_list.");
      TT_ENFORCE(value_tensor.shape(0) == 1 && value_tensor.shape(1) == sum_k, "The value_tensor shape 1 should be the sum of seq_len_list.");
      TT_ENFORCE(key_tensor.shape(2) == H && value_tensor.shape(2) == H, "key_tensor and value_tensor must be [1, sum_key_len, hidden]");
    } else {
      TT_ENFORCE_EQ(key_tensor.shape(0), B, "key_tensor and query_tensor disagree on the batch size");
      TT_ENFORCE(key_tensor.shape(1) == value_tensor.shape(1) && key_tensor.shape(2) == H && value_tensor.shape(2) == H &&
                     value_tensor.shape(0) == B,
                 "key_tensor and value_tensor must both be [batch, key_len, hidden]");
    }
    SameTypeDevice(key_tensor, k_.weight(), "attention");
    SameTypeDevice(value_tensor, v_.weight(), "attention");
    const int64_t Lk = packed ? *std::max_element(k_lens->begin(), k_lens->end()) : key_tensor.shape(1);  // padded key length
    const int64_t Tk = key_tensor.rows();
    if (memory_keys) { k = memory_keys; v = memory_values; }
    Tensor k_lin(nullptr), v_lin(nullptr);
    k_lin.Reshape(x.dtype(), {Tk, H}, kDLCUDA, dev, "context/gemm2/k_out1/Reshape");
    v_lin.Reshape(x.dtype(), {Tk, H}, kDLCUDA, dev, "context/gemm1/v_out1/Reshape");
    k_.Forward(key_tensor, Tk, TTB_EPI_NONE, nullptr, k_lin.raw_mut(), is_trans_weight, "context/gemm1");
    v_.Forward(value_tensor, Tk, TTB_EPI_NONE, nullptr, v_lin.raw_mut(), is_trans_weight, "context/gemm2");
    k->Reshape(x.dtype(), {B, heads, Lk, d}, kDLCUDA, dev, "context/keys/AddBiasTransposeForScore/Reshape");
    v->Reshape(x.dtype(), {B, heads, Lk, d}, kDLCUDA, dev, "context/values/AddBiasTransposeForScore/Reshape");
    Check(ttb_add_bias_transpose_for_score_pad(c, dt, k_lin.raw(), k_.bias().raw(), cu_k.get(), B, Lk, heads, d, k->raw_mut()), c,
          "context/keys/AddBiasTransposeForScore");
    Check(ttb_add_bias_transpose_for_score_pad(c, dt, v_lin.raw(), v_.bias().raw(), cu_k.get(), B, Lk, heads, d, v->raw_mut()), c,
          "context/values/AddBiasTransposeForScore");
  }
  const int64_t Lk = k->shape(2);

  // 3) scores, mask + softmax, weighted values
  Tensor scores_local(nullptr), ctx_heads(nullptr), context(nullptr);
  Tensor* scores = att_score ? att_score : &scores_local;
  scores->Reshape(x.dtype(), {B, heads, Lq, Lk}, kDLCUDA, dev, "batch_gemm3/Reshape");
  Check(ttb_batch_matmul(c, dt, q.raw(), 0, k->raw(), 1, B * heads, Lq, Lk, d, scale, 0.0f, scores->raw_mut()), c, "batch_gemm3");
  const float* mask = nullptr;
  int is2d = 1;
  Tensor pad_mask(nullptr);
  if (attention_mask.is_null() && packed) {
    // no mask tensor: keys beyond each sequence's own length are padding; the [B, 1, maxLk] additive mask the reference's
    // Python layer builds for this case (modeling_smart_pad.py:95-110)
    std::vector<float> host_mask((size_t)(B * Lk), 0.f);
    for (int64_t b = 0; b < B; ++b)
      for (int64_t l = (*k_lens)[b]; l < Lk; ++l) host_mask[b * Lk + l] = -1e9f;
    float* dm = pad_mask.Reshape<float>({B, 1, Lk}, kDLCUDA, dev, "context/pad_mask");
    Check(ttb_memcpy_h2d(c, dm, host_mask.data(), host_mask.size() * sizeof(float)), c, "context/pad_mask");
    mask = dm;
  }
  if (!attention_mask.is_null()) {
    TT_ENFORCE(attention_mask.on_gpu() && core::SameType(attention_mask.dtype(), core::kFloat32),
               "the attention mask must be an fp32 tensor on the GPU");
    TT_ENFORCE_EQ(attention_mask.shape(-1), Lk, "attention mask width must equal the key length");
    mask = attention_mask.data<float>();
    is2d = MaskIs2D(attention_mask) ? 1 : 0;
    if (!is2d) TT_ENFORCE_EQ(attention_mask.shape(-2), Lq, "a [B, Lq, Lk] attention mask must have one row per query");
  }
  Check(ttb_mask_softmax(c, dt, scores->raw_mut(), mask, B, heads, Lq, Lk, 1.0f, is2d), c, "ApplyMaskAndSoftmax");
  ctx_heads.Reshape(x.dtype(), {B, heads, Lq, d}, kDLCUDA, dev, "ApplyMaskAndSoftmax/Reshape");
  Check(ttb_batch_matmul(c, dt, scores->raw(), 0, v->raw(), 0, B * heads, Lq, d, Lk, 1.0f, 0.0f, ctx_heads.raw_mut()), c, "batch_gemm4");
  context.Reshape(x.dtype(), {T, H}, kDLCUDA, dev, "batch_gemm4/Reshape");
  Check(ttb_transpose_for_score_pad(c, dt, ctx_heads.raw(), cu_q.get(), B, Lq, heads, d, context.raw_mut()), c, "TransposeForScore");

  Finish(context, x, T, output, post_layernorm, post_add_input, is_trans_weight);
}

// ===================================================================================================
// feed-forward, pooler, pooling, masks
// ===================================================================================================
void BertIntermediate::EnforceShapeAndType() const {
  TT_ENFORCE_EQ(dense_.weight().n_dim(), 2, "dense weight must be matrix");
  TT_ENFORCE_EQ(dense_.bias().n_dim(), 1, "dense bias must be vector");
  TT_ENFORCE_EQ(dense_.weight().shape(1), dense_.bias().shape(0), "weight and bias shape mismatch");
}

void BertIntermediate::operator()(const Tensor& input_tensor, Tensor* output_tensor) const {
  TT_ENFORCE(output_tensor, "The output tensor should not be nullptr.");
  FloatType(input_tensor, "BertIntermediate input");
  const int dt = core::ToTTBDtype(input_tensor.dtype());
  const auto shape = WithLast(input_tensor, dense_.out_dim(false));
  output_tensor->Reshape(input_tensor.dtype(), shape, kDLCUDA, input_tensor.device_id(), "BertIntermediate/Reshape");
  void* out = output_tensor->raw_mut();
  void* lo = nullptr;
  if (PreciseMode(dt) && input_tensor.lo() && !dense_.use_int8())  // the activation leaves as two planes, like it came
    lo = output_tensor->NewExtras().lo.Reshape(input_tensor.dtype(), shape, kDLCUDA, input_tensor.device_id(), "precise/lo_plane");
  // int8 (per-row scheme): BertOutput's Linear takes this activation as int8, so it leaves with its int8 form attached
  Tensor* q8 = dense_.int8_mode() == PackedLinear::kInt8PerRow ? output_tensor : nullptr;
  dense_.Forward(input_tensor, input_tensor.rows(), TTB_EPI_BIAS_GELU, nullptr, out, false, "BertIntermediate", 0, lo, false, q8);
}

void BertOutput::EnforceShapeAndType() const {
  TT_ENFORCE_EQ(dense_.weight().n_dim(), 2, "dense weight must be matrix");
  TT_ENFORCE_EQ(dense_.bias().n_dim(), 1, "dense bias must be vector");
  TT_ENFORCE_EQ(dense_.weight().shape(1), dense_.bias().shape(0), "weight and bias shape mismatch");
  TT_ENFORCE_EQ(layer_norm_weight_.shape(0), dense_.weight().shape(1), "layer norm width mismatch");
}

void BertOutput::operator()(const Tensor& hidden_states, const Tensor& input_tensor, Tensor* output_tensor) const {
  TT_ENFORCE(output_tensor, "The output tensor should not be nullptr.");
  const int dt = FloatType(hidden_states, "BertOutput input");
  SameTypeDevice(hidden_states, input_tensor, "BertOutput");
  const int64_t M = hidden_states.rows(), N = dense_.out_dim(false);
  TT_ENFORCE_EQ(input_tensor.numel(), M * N, "BertOutput: residual shape mismatch");
  ttb_ctx* c = DeviceContext(hidden_states.device_id());
  output_tensor->Reshape(hidden_states.dtype(), WithLast(hidden_states, N), kDLCUDA, hidden_states.device_id(), "BertOutput/Reshape");
  if (dt == TTB_F32) {
    dense_.Forward(hidden_states, M, TTB_EPI_NONE, nullptr, output_tensor->raw_mut(), false, "BertOutput/MatMul");
    Check(ttb_add_bias_layernorm(c, dt, output_tensor->raw_mut(), input_tensor.raw(), dense_.bias().raw(), layer_norm_weight_.raw(),
                                 layer_norm_bias_.raw(), M, N, 1e-12f),
          c, "BertOutput/AddBiasLayerNorm");
  } else if (PreciseMode(dt) && input_tensor.f32() && !dense_.use_int8()) {
    Tensor sum(nullptr);
    float* s = sum.Reshape<float>({M, N}, kDLCUDA, hidden_states.device_id(), "BertOutput/fp32_sum");
    dense_.Forward(hidden_states, M, TTB_EPI_BIAS_RESIDUAL, input_tensor.f32()->raw(), s, false, "BertOutput/MatMul", 0, nullptr, true);
    LayerNormPlanes(c, true, s, output_tensor, layer_norm_weight_, layer_norm_bias_, M, N, 1e-12f, true, "BertOutput/AddBiasLayerNorm");
  } else {
    if (dense_.int8_mode() == PackedLinear::kInt8PerRow) {
      dense_.Forward(hidden_states, M, TTB_EPI_BIAS_RESIDUAL, input_tensor.raw(), output_tensor->raw_mut(), false, "BertOutput/MatMul");
      LayerNormWithInt8(c, output_tensor, layer_norm_weight_, layer_norm_bias_, M, N, 1e-12f, "BertOutput/AddBiasLayerNorm");
    } else {
      dense_.ForwardLayerNorm(hidden_states, M, input_tensor.raw(), layer_norm_weight_, layer_norm_bias_, 1e-12f, output_tensor->raw_mut(), false,
                              "BertOutput/MatMul");
    }
  }
}

namespace {
// out = LN(residual + act_in . W2 + b2) with W2's bias and the residual in the GEMM epilogue (16-bit) or in the
// AddBiasLayerNorm kernel (fp32, the reference's sequence).
void ProjectAddNorm(const PackedLinear& dense, const Tensor& act_in, const Tensor& residual, const Tensor& gamma, const Tensor& beta,
                    bool is_trans, Tensor* out, const char* name) {
  const int dt = FloatType(act_in, name);
  const int64_t M = act_in.rows(), N = dense.out_dim(is_trans);
  TT_ENFORCE_EQ(residual.numel(), M * N, "%s: residual shape mismatch", name);
  ttb_ctx* c = DeviceContext(act_in.device_id());
  out->Reshape(act_in.dtype(), ShapeOf(residual), kDLCUDA, act_in.device_id(), name);
  if (dt == TTB_F32) {
    dense.Forward(act_in, M, TTB_EPI_NONE, nullptr, out->raw_mut(), is_trans, name);
    Check(ttb_add_bias_layernorm(c, dt, out->raw_mut(), residual.raw(), dense.bias().raw(), gamma.raw(), beta.raw(), M, N, 1e-12f), c, name);
  } else if (PreciseMode(dt) && residual.f32() && !dense.use_int8()) {
    Tensor sum(nullptr);
    float* s = sum.Reshape<float>({M, N}, kDLCUDA, act_in.device_id(), "fp32_sum");
    dense.Forward(act_in, M, TTB_EPI_BIAS_RESIDUAL, residual.f32()->raw(), s, is_trans, name, 0, nullptr, true);
    LayerNormPlanes(c, true, s, out, gamma, beta, M, N, 1e-12f, true, name);
  } else {
    dense.ForwardLayerNorm(act_in, M, residual.raw(), gamma, beta, 1e-12f, out->raw_mut(), is_trans, name);
  }
}
}  // namespace

void DistrillFFN::operator()(const Tensor& x, Tensor* output, bool is_trans_weight) const {
  TT_ENFORCE(output, "The output tensor should not be nullptr.");
  FloatType(x, "DistrillFFN input");
  SameTypeDevice(x, dense1_.weight(), "DistrillFFN");
  TT_ENFORCE_EQ(dense1_.in_dim(is_trans_weight), x.shape(-1), "dense weight and input tensor should have the same model_dim.");
  Tensor inter(nullptr);
  inter.Reshape(x.dtype(), {x.rows(), dense1_.out_dim(is_trans_weight)}, kDLCUDA, x.device_id(), "FFN/gemm0/Reshape");
  void* inter_ptr = inter.raw_mut();
  void* inter_lo = nullptr;
  if (PreciseMode(core::ToTTBDtype(x.dtype())) && x.lo())
    inter_lo = inter.NewExtras().lo.Reshape(x.dtype(), ShapeOf(inter), kDLCUDA, x.device_id(), "precise/lo_plane");
  dense1_.Forward(x, x.rows(), TTB_EPI_BIAS_GELU, nullptr, inter_ptr, is_trans_weight, "FFN/gemm0", 0, inter_lo);
  ProjectAddNorm(dense2_, inter, x, layer_norm_weight_, layer_norm_bias_, is_trans_weight, output, "FFN/gemm1");
}

void AlbertLayer::EnforceShapeAndType() const {
  TT_ENFORCE_EQ(dense_.weight().n_dim(), 2, "dense weight must be matrix");
  TT_ENFORCE_EQ(dense_.bias().n_dim(), 1, "dense bias must be vector");
  TT_ENFORCE_EQ(dense_.weight().shape(1), dense_.bias().shape(0), "weight and bias shape mismatch");
  TT_ENFORCE_EQ(dense_output_.weight().shape(0), dense_.weight().shape(1), "the two dense layers do not chain");
}

void AlbertLayer::operator()(const Tensor& x, Tensor* hidden_output, Tensor* output) const {
  TT_ENFORCE(hidden_output && output, "The output tensors should not be nullptr.");
  FloatType(x, "AlbertLayer input");
  SameTypeDevice(x, dense_.weight(), "AlbertLayer");
  hidden_output->Reshape(x.dtype(), WithLast(x, dense_.out_dim(false)), kDLCUDA, x.device_id(), "AlbertLayer/Reshape");
  void* hid_ptr = hidden_output->raw_mut();
  void* hid_lo = nullptr;
  if (PreciseMode(core::ToTTBDtype(x.dtype())) && x.lo())
    hid_lo = hidden_output->NewExtras().lo.Reshape(x.dtype(), ShapeOf(*hidden_output), kDLCUDA, x.device_id(), "precise/lo_plane");
  dense_.Forward(x, x.rows(), TTB_EPI_BIAS_GELU, nullptr, hid_ptr, false, "AlbertLayer/gemm0", 0, hid_lo);
  ProjectAddNorm(dense_output_, *hidden_output, x, layer_norm_weight_, layer_norm_bias_, false, output, "AlbertLayer/gemm1");
}

void BertPooler::EnforceShapeAndType() const {
  TT_ENFORCE_EQ(dense_.weight().n_dim(), 2, "dense weight must be matrix");
  TT_ENFORCE_EQ(dense_.bias().n_dim(), 1, "dense bias must be vector");
  TT_ENFORCE_EQ(dense_.weight().shape(1), dense_.bias().shape(0), "weight and bias shape mismatch %lld, %lld",
                (long long)dense_.weight().shape(1), (long long)dense_.bias().shape(0));
}

void BertPooler::operator()(const Tensor& input_tensor, Tensor* output_tensor) const {
  TT_ENFORCE_EQ(input_tensor.n_dim(), 2, "input's dim should be 2, not %zu", input_tensor.n_dim());
  FloatType(input_tensor, "BertPooler input");
  output_tensor->Reshape(input_tensor.dtype(), {input_tensor.shape(0), dense_.out_dim(false)}, kDLCUDA, input_tensor.device_id(),
                         "BertPooler");
  dense_.Forward(input_tensor, input_tensor.shape(0), TTB_EPI_BIAS_TANH, nullptr, output_tensor->raw_mut(), false, "BertPooler");
}

SequencePool::SequencePool(const std::string& pool_type) {
  if (pool_type == "First") pool_type_ = TTB_POOL_FIRST;
  else if (pool_type == "Last") pool_type_ = TTB_POOL_LAST;
  else if (pool_type == "Mean") pool_type_ = TTB_POOL_MEAN;
  else if (pool_type == "Max") pool_type_ = TTB_POOL_MAX;
  else TT_THROW("The input pool type (%s) is not supported.", pool_type.c_str());
}

void SequencePool::operator()(const Tensor& input, Tensor* output) const {
  TT_ENFORCE_EQ(input.n_dim(), 3, "The input's dim should be 3, but the input's dim is %zu", input.n_dim());
  const int dt = FloatType(input, "SequencePool input");
  ttb_ctx* c = DeviceContext(input.device_id());
  output->Reshape(input.dtype(), {input.shape(0), input.shape(2)}, kDLCUDA, input.device_id(), "SequencePool/Reshape");
  Check(ttb_seq_pool(c, dt, input.raw(), input.shape(0), input.shape(1), input.shape(2), pool_type_, output->raw_mut()), c, "SeqPool");
}

void SequencePool::Packed(const Tensor& input, const std::vector<int64_t>& seq_lens, Tensor* output) const {
  const int dt = FloatType(input, "SequencePool input");
  const int dev = input.device_id();
  ttb_ctx* c = DeviceContext(dev);
  const int64_t B = (int64_t)seq_lens.size(), H = input.shape(-1);
  output->Reshape(input.dtype(), {B, H}, kDLCUDA, dev, "SequencePool/Reshape");
  const core::CuSeqlensHandle cu = core::CuSeqlens(dev, seq_lens);
  Check(ttb_seq_pool_varlen(c, dt, input.raw(), cu.get(), B, H, pool_type_, output->raw_mut()), c, "SeqPool/packed");
}

void PrepareBertMasks::operator()(const Tensor& inputs, Tensor* att_mask, Tensor* seq_type, Tensor* position_ids,
                                  Tensor* extended_attention_mask) const {
  TT_ENFORCE_EQ(inputs.n_dim(), 2, "inputs must be [batch, seq_len]");
  TT_ENFORCE(inputs.on_gpu(), "inputs must be on the GPU: this runtime has no CPU path");
  const int64_t B = inputs.shape(0), L = inputs.shape(1);
  const int dev = inputs.device_id();
  ttb_ctx* c = DeviceContext(dev);
  int64_t *pos_out = nullptr, *type_out = nullptr, *mask_out = nullptr;
  const int64_t* mask_in = nullptr;
  if (position_ids->is_null()) pos_out = position_ids->Reshape<int64_t>({B, L}, kDLCUDA, dev, "PrepareBertMasks/possitionids/Reshape");
  if (seq_type->is_null()) type_out = seq_type->Reshape<int64_t>({B, L}, kDLCUDA, dev, "PrepareBertMasks/seqids/Reshape");
  if (att_mask->is_null()) mask_out = att_mask->Reshape<int64_t>({B, L}, kDLCUDA, dev, "PrepareBertMasks/attmask/Reshape");
  else mask_in = att_mask->data<int64_t>();
  float* ext = extended_attention_mask->Reshape<float>({B, 1, 1, L}, kDLCUDA, dev, "PrepareBertMasks/extendedattnmask/Reshape");
  Check(ttb_prepare_bert_masks(c, B, L, mask_in, mask_out, type_out, pos_out, ext), c, "PrepareBertMasks");
}

void PositionwiseFeedForward::set_activation(const std::string& act) {
  if (act == "relu") act_ = TTB_ACT_RELU;
  else if (act == "gelu") act_ = TTB_ACT_GELU;
  else TT_THROW("activation must be relu or gelu");
}

void PositionwiseFeedForward::operator()(const Tensor& x, Tensor* output, bool is_trans_weight) const {
  const int dt = FloatType(x, "FFN input");
  const int dev = x.device_id();
  ttb_ctx* c = DeviceContext(dev);
  const int64_t M = x.rows(), H = x.shape(-1), F = dense1_.out_dim(is_trans_weight);
  TT_ENFORCE_EQ(dense1_.in_dim(is_trans_weight), H, "dense weight and input tensor should have the same model_dim.");
  Tensor normed(nullptr), inter(nullptr);
  normed.Reshape(x.dtype(), ShapeOf(x), kDLCUDA, dev, "FFN/LayerNorm/Reshape");
  inter.Reshape(x.dtype(), {M, F}, kDLCUDA, dev, "FFN/inter/Reshape");
  if (PreciseMode(dt) && act_ == TTB_ACT_GELU) {
    // pre-LN block of a bf16 model: normalise the fp32 stream into two operand planes, keep the GELU output as two
    // planes, add into the fp32 stream and leave its 16-bit copy for the caller
    LayerNormPlanes(c, x.f32() != nullptr, x.f32() ? x.f32()->raw() : x.raw(), &normed, layer_norm_weight_, layer_norm_bias_, M, H, eps_, false,
                    "FFN/LayerNorm");
    void* inter_ptr = inter.raw_mut();
    void* inter_lo = inter.NewExtras().lo.Reshape(x.dtype(), {M, F}, kDLCUDA, dev, "precise/lo_plane");
    dense1_.Forward(normed, M, TTB_EPI_BIAS_GELU, nullptr, inter_ptr, is_trans_weight, "FFN/gemm0", 0, inter_lo);
    output->Reshape(x.dtype(), ShapeOf(x), kDLCUDA, dev, "FFN/Reshape");
    if (x.f32()) {
      void* pub = output->raw_mut();
      float* s = output->NewExtras().f32.Reshape<float>(ShapeOf(x), kDLCUDA, dev, "precise/residual_stream");
      dense2_.Forward(inter, M, TTB_EPI_BIAS_RESIDUAL, x.f32()->raw(), s, is_trans_weight, "FFN/gemm1", 0, nullptr, true);
      CastFromF32(c, s, dt, pub, M, H, "FFN/public_copy");
    } else {
      dense2_.Forward(inter, M, TTB_EPI_BIAS_RESIDUAL, x.raw(), output->raw_mut(), is_trans_weight, "FFN/gemm1");
    }
    return;
  }
  Check(ttb_layernorm(c, dt, x.raw(), normed.raw_mut(), layer_norm_weight_.raw(), layer_norm_bias_.raw(), M, H, eps_), c, "FFN/LayerNorm");
  if (act_ == TTB_ACT_GELU) {
    dense1_.Forward(normed, M, TTB_EPI_BIAS_GELU, nullptr, inter.raw_mut(), is_trans_weight, "FFN/gemm0");
  } else {
    dense1_.Forward(normed, M, TTB_EPI_NONE, nullptr, inter.raw_mut(), is_trans_weight, "FFN/gemm0");
    Check(ttb_add_bias_act(c, dt, inter.raw_mut(), dense1_.bias().raw(), M, F, TTB_ACT_RELU), c, "FFN/AddBiasAct");
  }
  output->Reshape(x.dtype(), ShapeOf(x), kDLCUDA, dev, "FFN/Reshape");
  dense2_.Forward(inter, M, TTB_EPI_BIAS_RESIDUAL, x.raw(), output->raw_mut(), is_trans_weight, "FFN/gemm1");
}

void FusedAddBiasGELU::operator()(Tensor* t) const {
  const int dt = FloatType(*t, "FusedAddBiasGELU input");
  ttb_ctx* c = DeviceContext(t->device_id());
  Check(ttb_add_bias_act(c, dt, t->raw_mut(), bias_.raw(), t->rows(), t->shape(-1), TTB_ACT_GELU), c, "FusedAddBiasGELU");
}

void FusedAddBiasLayerNorm::operator()(const Tensor& input_tensor, Tensor* output_tensor) const {
  const int dt = FloatType(*output_tensor, "FusedAddBiasLayerNorm output");
  SameTypeDevice(input_tensor, *output_tensor, "FusedAddBiasLayerNorm");
  ttb_ctx* c = DeviceContext(output_tensor->device_id());
  Check(ttb_add_bias_layernorm(c, dt, output_tensor->raw_mut(), input_tensor.raw(), bias_.raw(), norm_weight_.raw(), norm_bias_.raw(),
                               output_tensor->rows(), output_tensor->shape(-1), 1e-12f),
        c, "FusedAddBiasLayerNorm");
}

void LayerNorm::operator()(const Tensor& input, Tensor* output) const {
  const int dt = FloatType(input, "LayerNorm input");
  ttb_ctx* c = DeviceContext(input.device_id());
  if (PreciseMode(dt) && output != &input) {  // the final norm of a pre-LN bf16 model reads the fp32 stream when there is one
    const bool f = input.f32() != nullptr;
    const void* in = f ? input.f32()->raw() : input.raw();
    const int64_t rows = input.rows(), width = input.shape(-1);
    const auto shape = ShapeOf(input);
    output->Reshape(input.dtype(), shape, kDLCUDA, input.device_id(), "LayerNorm/Reshape");
    LayerNormPlanes(c, f, in, output, gamma_, beta_, rows, width, eps_, false, "LayerNorm");
    return;
  }
  output->Reshape(input.dtype(), ShapeOf(input), kDLCUDA, input.device_id(), "LayerNorm/Reshape");
  Check(ttb_layernorm(c, dt, input.raw(), output->raw_mut(), gamma_.raw(), beta_.raw(), input.rows(), input.shape(-1), eps_), c, "LayerNorm");
}

void TokenPositionEmbedding::operator()(const Tensor& input_ids, Tensor* output, int64_t position_offset) const {
  TT_ENFORCE_EQ(input_ids.n_dim(), 2, "The input ids should be a matrix with shape [BatchSize, SeqLen].");
  const int dt = FloatType(token_, "token embeddings");
  TT_ENFORCE(input_ids.on_gpu(), "input ids must be on the GPU");
  const int64_t B = input_ids.shape(0), L = input_ids.shape(1), H = token_.shape(1);
  const int dev = input_ids.device_id();
  ttb_ctx* c = DeviceContext(dev);
  Tensor pos(nullptr);
  int64_t* pos_ids = pos.Reshape<int64_t>({B, L}, kDLCUDA, dev, "TokenPositionEmbedding/positions");
  Check(ttb_prepare_bert_masks(c, B, L, nullptr, nullptr, nullptr, pos_ids, nullptr), c, "TokenPositionEmbedding/positions");
  output->Reshape(token_.dtype(), {B, L, H}, kDLCUDA, dev, "TokenPositionEmbedding/Reshape");
  Check(ttb_lookup_embedding(c, dt, output->raw_mut(), token_.raw(), input_ids.data<int64_t>(), B * L, H, token_.shape(0), 0), c,
        "TokenPositionEmbedding/token");
  TT_ENFORCE(position_offset >= 0 && position_offset + L <= position_.shape(0), "positions %lld..%lld exceed the %lld the model has",
             (long long)position_offset, (long long)(position_offset + L - 1), (long long)position_.shape(0));
  const char* table = static_cast<const char*>(position_.raw()) + (size_t)position_offset * (size_t)H * (dt == TTB_F32 ? 4 : 2);
  Check(ttb_lookup_embedding(c, dt, output->raw_mut(), table, pos_ids, B * L, H, position_.shape(0) - position_offset, 1), c,
        "TokenPositionEmbedding/position");
  if (PreciseMode(dt)) {
    // start the fp32 residual stream of a bf16 model from the embedding sum (its one rounding is 2^-9 of a value of the
    // embeddings' size, far below what the blocks add)
    const void* pub = output->raw();
    float* f = output->NewExtras().f32.Reshape<float>({B, L, H}, kDLCUDA, dev, "precise/residual_stream");
    Check(ttb_prepack_weight(c, dt, pub, 1, H, B * L, TTB_F32, f), c, "TokenPositionEmbedding/residual_stream");
  }
}

void Linear::operator()(const Tensor& input, Tensor* output) const {
  FloatType(input, "Linear input");
  const int dt = core::ToTTBDtype(input.dtype());
  const int64_t N = dense_.out_dim(is_trans_), M = input.rows();
  output->Reshape(input.dtype(), WithLast(input, N), kDLCUDA, input.device_id(), "Linear/Reshape");
  if (dt != TTB_F32 && N % 8 != 0) {
    // An output row that is not a multiple of 16 bytes (e.g. a 50257-wide vocabulary) would force the GEMM onto scalar
    // stores. Compute into a row-padded scratch with the fast epilogue, then compact: one extra pass over the output
    // at copy bandwidth instead of a several-times slower GEMM.
    const int64_t Np = (N + 7) / 8 * 8;
    ttb_ctx* c = DeviceContext(input.device_id());
    Tensor padded(nullptr);
    padded.Reshape(input.dtype(), {M, Np}, kDLCUDA, input.device_id(), "Linear/padded");
    dense_.Forward(input, M, TTB_EPI_BIAS, nullptr, padded.raw_mut(), is_trans_, "Linear", Np);
    Check(ttb_copy_2d(c, output->raw_mut(), (size_t)N * 2, padded.raw(), (size_t)Np * 2, (size_t)N * 2, (size_t)M), c, "Linear/compact");
    return;
  }
  dense_.Forward(input, M, TTB_EPI_BIAS, nullptr, output->raw_mut(), is_trans_, "Linear");
}

void Linear::Padded(const Tensor& input, Tensor* output) const {
  FloatType(input, "Linear input");
  const int dt = core::ToTTBDtype(input.dtype());
  const int64_t N = Width(), Np = PaddedWidth(), M = input.rows();
  if (dt == TTB_F32 || Np == N) {  // nothing to gain: the plain path already stores whole rows
    (*this)(input, output);
    return;
  }
  output->Reshape(input.dtype(), WithLast(input, Np), kDLCUDA, input.device_id(), "Linear/Reshape");
  dense_.Forward(input, M, TTB_EPI_BIAS, nullptr, output->raw_mut(), is_trans_, "Linear", Np);
}

}  // namespace layers
}  // namespace turbo_transformers
