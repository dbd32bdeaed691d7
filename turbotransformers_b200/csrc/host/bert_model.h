// A BERT encoder that runs from an `.npz` archive with no Python in the process: the class of the reference's C++ example
// (example/cpp/bert_model.h:26-44, bert_model.cpp:33-254) over this library's layer classes. Same constructor arguments and
// call signature; `dtype` ("float32" | "float16" | "bfloat16") and `device_id` are additions.
//
//   fp32 models   : the reference's own sequence - ids padded to the longest request, PrepareBertMasks, embedding, the
//                   encoder layers with the additive mask - on exact-precision kernels.
//   16-bit models : requests are packed back to back (no padding, no mask tensor) and run through the tensor-core path;
//                   the result is scattered into the reference's padded layout with zeros at padding positions.
// One object serves one device; objects on different devices may be driven from different host threads.
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "dlpack_abi.h"

namespace turbo_transformers {
namespace layers {
namespace types {
enum class PoolType { kMax = 0, kMean, kFirst, kLast };
}  // namespace types
}  // namespace layers
}  // namespace turbo_transformers

using PoolType = turbo_transformers::layers::types::PoolType;

class BertModel {
 public:
  BertModel(const std::string& filename, DLDeviceType device_type, size_t n_layers, int64_t n_heads,
            const std::string& dtype = "float32", int device_id = 0);
  ~BertModel();

  // inputs[b] = token ids of request b. position_ids / segment_ids may be empty (positions 0..L-1, segment 0).
  // use_pooler = false: the final hidden states, [batch, longest, hidden] row-major;
  // use_pooler = true : tanh(W . pool(hidden) + b), [batch, hidden].
  std::vector<float> operator()(const std::vector<std::vector<int64_t>>& inputs, const std::vector<std::vector<int64_t>>& position_ids,
                                const std::vector<std::vector<int64_t>>& segment_ids, PoolType pooling = PoolType::kFirst,
                                bool use_pooler = false) const;
  int64_t hidden_size() const;

 private:
  struct Impl;
  std::unique_ptr<Impl> m_;
};
