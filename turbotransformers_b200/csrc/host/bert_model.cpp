#include "bert_model.h"

#include <algorithm>
#include <cstring>
#include <numeric>

#include "layers.h"
#include "npz.h"

using namespace turbo_transformers;
using core::Tensor;

namespace {

DLDataType ParseDtype(const std::string& s) {
  if (s == "float32" || s == "fp32") return {kDLFloat, 32, 1};
  if (s == "float16" || s == "fp16" || s == "half") return {kDLFloat, 16, 1};
  if (s == "bfloat16" || s == "bf16") return {kDLBfloat, 16, 1};
  TT_THROW("dtype must be float32, float16 or bfloat16, not %s", s.c_str());
}

const char* PoolName(PoolType p) {
  switch (p) {
    case PoolType::kMax: return "Max";
    case PoolType::kMean: return "Mean";
    case PoolType::kFirst: return "First";
    case PoolType::kLast: return "Last";
  }
  return "First";
}

float HalfToFloat(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {  // subnormal: renormalise
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while (!(man & 0x400u));
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// Device tensor (fp32 / fp16 / bf16) -> host floats.
void ToHostFloats(const Tensor& t, float* dst) {
  ttb_ctx* c = core::DeviceContext(t.device_id());
  const int64_t n = t.numel();
  const DLDataType dt = t.dtype();
  if (dt.bits == 32) {
    core::Check(ttb_memcpy_d2h(c, dst, t.raw(), (size_t)n * 4), c, "BertModel/copy out");
    return;
  }
  std::vector<uint16_t> raw((size_t)n);
  core::Check(ttb_memcpy_d2h(c, raw.data(), t.raw(), (size_t)n * 2), c, "BertModel/copy out");
  if (dt.code == kDLBfloat) {
    for (int64_t i = 0; i < n; ++i) {
      const uint32_t bits = (uint32_t)raw[(size_t)i] << 16;
      std::memcpy(&dst[i], &bits, 4);
    }
  } else {
    for (int64_t i = 0; i < n; ++i) dst[i] = HalfToFloat(raw[(size_t)i]);
  }
}

void UploadIds(const std::vector<int64_t>& host, const std::vector<int64_t>& shape, int dev, Tensor* t, const char* name) {
  ttb_ctx* c = core::DeviceContext(dev);
  t->Reshape<int64_t>(shape, kDLCUDA, dev, name);
  core::Check(ttb_memcpy_h2d(c, t->raw_mut(), host.data(), host.size() * sizeof(int64_t)), c, name);
}

struct BertLayer {
  BertLayer(loaders::NPZLoader p, int64_t n_heads)
      : attention(p["attention.qkv.weight"], p["attention.qkv.bias"], p["attention.output.dense.weight"], p["attention.output.dense.bias"],
                  p["attention.output.LayerNorm.weight"], p["attention.output.LayerNorm.bias"], n_heads),
        intermediate(p["intermediate.dense.weight"], p["intermediate.dense.bias"]),
        output(p["output.dense.weight"], p["output.dense.bias"], p["output.LayerNorm.weight"], p["output.LayerNorm.bias"]) {}
  layers::BertAttention attention;
  layers::BertIntermediate intermediate;
  layers::BertOutput output;
};

}  // namespace

struct BertModel::Impl {
  Impl(const std::string& filename, DLDeviceType device_type, size_t n_layers, int64_t n_heads, const std::string& dtype, int device_id)
      : dtype_(ParseDtype(dtype)), dev_(device_id) {
    TT_ENFORCE(device_type == kDLCUDA, "BertModel runs on a CUDA device (there is no CPU path)");
    loaders::npz_t npz = loaders::npz_load(filename);
    loaders::NPZMapView root("", &npz);
    {
      loaders::NPZLoader p(root.Sub("embeddings"), kDLCUDA, dev_, dtype_);
      embedding_.reset(new layers::BERTEmbedding(p["word_embeddings.weight"], p["position_embeddings.weight"],
                                                 p["token_type_embeddings.weight"], p["LayerNorm.weight"], p["LayerNorm.bias"]));
      hidden_ = npz.at("embeddings.word_embeddings.weight").shape.at(1);
    }
    for (size_t i = 0; i < n_layers; ++i) {
      loaders::NPZLoader p(root.Sub("encoder.layer." + std::to_string(i)), kDLCUDA, dev_, dtype_);
      layers_.emplace_back(new BertLayer(p, n_heads));
    }
    if (root.IsExist("pooler")) {
      loaders::NPZLoader p(root.Sub("pooler"), kDLCUDA, dev_, dtype_);
      pooler_.reset(new layers::BertPooler(p["dense.weight"], p["dense.bias"]));
    }
  }

  std::vector<float> Run(const std::vector<std::vector<int64_t>>& inputs, const std::vector<std::vector<int64_t>>& position_ids,
                         const std::vector<std::vector<int64_t>>& segment_ids, PoolType pooling, bool use_pooler) const {
    const int64_t B = (int64_t)inputs.size();
    TT_ENFORCE(B > 0, "BertModel needs at least one request");
    TT_ENFORCE(position_ids.empty() || (int64_t)position_ids.size() == B, "Position ids should have the same batch size as input ids");
    TT_ENFORCE(segment_ids.empty() || (int64_t)segment_ids.size() == B, "Segment ids should have the same batch size as input ids");
    TT_ENFORCE(!use_pooler || pooler_, "the archive has no pooler parameters");
    std::vector<int64_t> lens((size_t)B);
    for (int64_t b = 0; b < B; ++b) lens[(size_t)b] = (int64_t)inputs[(size_t)b].size();
    const int64_t L = *std::max_element(lens.begin(), lens.end());
    TT_ENFORCE(L > 0, "every request is empty");
    const bool packed = dtype_.bits == 16 && position_ids.empty() && segment_ids.empty();
    return packed ? RunPacked(inputs, lens, L, pooling, use_pooler) : RunPadded(inputs, position_ids, segment_ids, lens, L, pooling, use_pooler);
  }

  // The reference's sequence (example/cpp/bert_model.cpp:131-236): pad, masks, embedding, layers with the additive mask.
  std::vector<float> RunPadded(const std::vector<std::vector<int64_t>>& inputs, const std::vector<std::vector<int64_t>>& position_ids,
                               const std::vector<std::vector<int64_t>>& segment_ids, const std::vector<int64_t>& lens, int64_t L,
                               PoolType pooling, bool use_pooler) const {
    const int64_t B = (int64_t)inputs.size();
    auto pad = [&](const std::vector<std::vector<int64_t>>& rows, int64_t fill) {
      std::vector<int64_t> flat((size_t)(B * L), fill);
      for (int64_t b = 0; b < B; ++b) {
        TT_ENFORCE((int64_t)rows[(size_t)b].size() <= L, "a row of ids is longer than its request");
        std::copy(rows[(size_t)b].begin(), rows[(size_t)b].end(), flat.begin() + b * L);
      }
      return flat;
    };
    std::vector<int64_t> mask((size_t)(B * L), 0);
    for (int64_t b = 0; b < B; ++b) std::fill(mask.begin() + b * L, mask.begin() + b * L + lens[(size_t)b], 1);
    Tensor ids(nullptr), att_mask(nullptr), seq_type(nullptr), pos(nullptr), ext_mask(nullptr);
    UploadIds(pad(inputs, 0), {B, L}, dev_, &ids, "BertModel/ids");
    UploadIds(mask, {B, L}, dev_, &att_mask, "BertModel/mask");
    if (!position_ids.empty()) UploadIds(pad(position_ids, 0), {B, L}, dev_, &pos, "BertModel/position ids");
    if (!segment_ids.empty()) UploadIds(pad(segment_ids, 0), {B, L}, dev_, &seq_type, "BertModel/segment ids");
    layers::PrepareBertMasks()(ids, &att_mask, &seq_type, &pos, &ext_mask);
    Tensor hidden(nullptr), att_out(nullptr), inter(nullptr);
    (*embedding_)(ids, pos, seq_type, &hidden);
    for (const auto& layer : layers_) {
      layer->attention(hidden, ext_mask, &att_out);
      layer->intermediate(att_out, &inter);
      layer->output(inter, att_out, &hidden);
    }
    std::vector<float> out;
    if (use_pooler) {
      Tensor pooled(nullptr), y(nullptr);
      layers::SequencePool(PoolName(pooling))(hidden, &pooled);
      (*pooler_)(pooled, &y);
      out.resize((size_t)y.numel());
      ToHostFloats(y, out.data());
    } else {
      out.resize((size_t)hidden.numel());
      ToHostFloats(hidden, out.data());
    }
    return out;
  }

  // 16-bit models: one packed [1, sum L, H] batch, no padding anywhere on the device.
  std::vector<float> RunPacked(const std::vector<std::vector<int64_t>>& inputs, const std::vector<int64_t>& lens, int64_t L, PoolType pooling,
                               bool use_pooler) const {
    const int64_t B = (int64_t)inputs.size();
    const int64_t T = std::accumulate(lens.begin(), lens.end(), (int64_t)0);
    std::vector<int64_t> flat;
    flat.reserve((size_t)T);
    for (const auto& r : inputs) flat.insert(flat.end(), r.begin(), r.end());
    Tensor ids(nullptr), hidden(nullptr), att_out(nullptr), inter(nullptr), no_mask(nullptr);
    UploadIds(flat, {T}, dev_, &ids, "BertModel/packed ids");
    embedding_->Packed(ids, lens, &hidden);
    for (const auto& layer : layers_) {
      layer->attention.Run(hidden, no_mask, &lens, &att_out, nullptr, false, true, false, false);
      layer->intermediate(att_out, &inter);
      layer->output(inter, att_out, &hidden);
    }
    std::vector<float> out;
    if (use_pooler) {
      Tensor pooled(nullptr), y(nullptr);
      layers::SequencePool(PoolName(pooling)).Packed(hidden, lens, &pooled);
      (*pooler_)(pooled, &y);
      out.resize((size_t)y.numel());
      ToHostFloats(y, out.data());
      return out;
    }
    std::vector<float> rows((size_t)(T * hidden_));
    ToHostFloats(hidden, rows.data());
    out.assign((size_t)(B * L * hidden_), 0.f);
    int64_t t0 = 0;
    for (int64_t b = 0; b < B; ++b) {
      std::copy(rows.begin() + t0 * hidden_, rows.begin() + (t0 + lens[(size_t)b]) * hidden_, out.begin() + b * L * hidden_);
      t0 += lens[(size_t)b];
    }
    return out;
  }

  DLDataType dtype_;
  int dev_;
  int64_t hidden_ = 0;
  std::unique_ptr<layers::BERTEmbedding> embedding_;
  std::vector<std::unique_ptr<BertLayer>> layers_;
  std::unique_ptr<layers::BertPooler> pooler_;
};

BertModel::BertModel(const std::string& filename, DLDeviceType device_type, size_t n_layers, int64_t n_heads, const std::string& dtype,
                     int device_id)
    : m_(new Impl(filename, device_type, n_layers, n_heads, dtype, device_id)) {}

BertModel::~BertModel() = default;

std::vector<float> BertModel::operator()(const std::vector<std::vector<int64_t>>& inputs, const std::vector<std::vector<int64_t>>& position_ids,
                                         const std::vector<std::vector<int64_t>>& segment_ids, PoolType pooling, bool use_pooler) const {
  return m_->Run(inputs, position_ids, segment_ids, pooling, use_pooler);
}

int64_t BertModel::hidden_size() const { return m_->hidden_; }
