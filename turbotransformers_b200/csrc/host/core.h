// Host runtime of the layer classes: exceptions, per-device contexts, and the DLPack-backed Tensor.
//
// Mirrors the reference's core/ API (turbo_transformers/core/tensor.h:117-354, enforce.h:41-85,
// cuda_device_context.h, allocator/allocator_api.h) so code written against it keeps compiling:
// same namespaces, class and method names. Differences, all on purpose:
//   * a Tensor carries any of fp32/fp16/bf16/int8/int64 (the reference was fp32/int64 only) and layers
//     dispatch on it;
//   * device memory comes from the stream-ordered pool behind the C ABI (ttb_alloc), one context per
//     device, instead of a process-wide cub caching allocator on device 0;
//   * CUDA failures raise EnforceNotMet (the reference printed and called exit(0)).
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <exception>
#include <memory>
#include <numeric>
#include <string>
#include <vector>

#include "dlpack_abi.h"
#include "ttb.h"

namespace turbo_transformers {
namespace core {

namespace details {
class EnforceNotMet : public std::exception {
 public:
  explicit EnforceNotMet(std::string msg) : msg_(std::move(msg)) {}
  const char* what() const noexcept override { return msg_.c_str(); }

 private:
  std::string msg_;
};
inline std::string Format(const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  return std::string(buf);
}
}  // namespace details

#define TT_THROW(...) throw ::turbo_transformers::core::details::EnforceNotMet(::turbo_transformers::core::details::Format(__VA_ARGS__))
#define TT_ENFORCE(cond, ...) \
  do {                        \
    if (!(cond)) TT_THROW("enforce failed: " #cond ": " __VA_ARGS__); \
  } while (0)
#define TT_ENFORCE_EQ(a, b, ...) TT_ENFORCE((a) == (b), __VA_ARGS__)
#define TT_ENFORCE_NE(a, b, ...) TT_ENFORCE((a) != (b), __VA_ARGS__)
#define TT_ENFORCE_GE(a, b, ...) TT_ENFORCE((a) >= (b), __VA_ARGS__)
#define TT_ENFORCE_LE(a, b, ...) TT_ENFORCE((a) <= (b), __VA_ARGS__)

// ---- per-device contexts (replaces the CUDADeviceContext singleton) ------------------------------
// The context of `device_id`, created on first use on the legacy default stream.
ttb_ctx* DeviceContext(int device_id);
// Points the device's context at another CUDA stream (a cudaStream_t; nullptr = legacy default stream).
void SetDeviceStream(int device_id, void* cuda_stream);
// Throws EnforceNotMet carrying ttb_last_error when `status` is not TTB_OK.
void Check(int status, ttb_ctx* ctx, const char* what);
// A device int32 [B+1] prefix-sum array for these sequence lengths; cached per device, so the 12 layers
// of one forward (and repeated shapes) share one table. The caller holds the handle until it has queued the last kernel
// that reads the array: eviction from the cache only drops the cache's own reference, and the array goes back to the
// pool (stream ordered) when the last holder lets go.
using CuSeqlensHandle = std::shared_ptr<const int32_t>;
CuSeqlensHandle CuSeqlens(int device_id, const std::vector<int64_t>& seq_lens);
// Same for B equal sequences of length L.
CuSeqlensHandle UniformCuSeqlens(int device_id, int64_t B, int64_t L);

// ---- dtype helpers --------------------------------------------------------------------------------
template <typename T> struct DataTypeTrait;
template <> struct DataTypeTrait<float> { static constexpr DLDataType value() { return {kDLFloat, 32, 1}; } };
template <> struct DataTypeTrait<int64_t> { static constexpr DLDataType value() { return {kDLInt, 64, 1}; } };
template <> struct DataTypeTrait<int32_t> { static constexpr DLDataType value() { return {kDLInt, 32, 1}; } };
template <> struct DataTypeTrait<int8_t> { static constexpr DLDataType value() { return {kDLInt, 8, 1}; } };
constexpr DLDataType kFloat32{kDLFloat, 32, 1}, kFloat16{kDLFloat, 16, 1}, kBFloat16{kDLBfloat, 16, 1}, kInt64{kDLInt, 64, 1},
    kInt8{kDLInt, 8, 1}, kInt32{kDLInt, 32, 1};
inline bool SameType(DLDataType a, DLDataType b) { return a.code == b.code && a.bits == b.bits; }
// ttb_dtype of a floating DLPack type, or -1.
int ToTTBDtype(DLDataType dt);

DLManagedTensor* NewDLPackTensor(const std::vector<int64_t>& shape, DLDeviceType device, int device_id, DLDataType dtype,
                                 const std::string& name);

// Whether bf16 models keep an fp32 residual stream and hi + lo activation planes between their layers (default on;
// TTB_BF16_PRECISE=0 or SetPreciseBF16(false) selects plain bf16 storage, which is faster and 8 bits accurate).
bool PreciseBF16();
void SetPreciseBF16(bool on);
// Whether fp32 models run their Linears on the tensor cores as three tf32 products (default on; TTB_FP32_GEMM=simt or
// SetFp32TensorCores(false) selects the exact-order CUDA-core GEMM).
bool Fp32TensorCores();
void SetFp32TensorCores(bool on);

struct TensorExtras;

class Tensor {
 public:
  // Takes ownership of `tensor` (nullptr makes a null Tensor), as core::Tensor(DLManagedTensor*) did.
  explicit Tensor(DLManagedTensor* tensor) : owned_(tensor) {
    if (tensor) view_ = tensor->dl_tensor;
  }
  Tensor(const Tensor&) = delete;
  Tensor& operator=(const Tensor&) = delete;
  Tensor(Tensor&& o) noexcept { MoveFrom(o); }
  Tensor& operator=(Tensor&& o) noexcept {
    if (this != &o) {
      Release();
      MoveFrom(o);
    }
    return *this;
  }
  ~Tensor() { Release(); }

  // Gives the DLManagedTensor away (the Tensor becomes null). A view cannot be exported.
  DLManagedTensor* ToDLPack();

  bool is_null() const { return !owned_ && !is_view_; }
  size_t n_dim() const { return is_null() ? 0 : (size_t)view_.ndim; }
  int64_t shape(int pos) const;  // negative positions count from the end
  int64_t numel() const;
  size_t capacity_bytes() const;  // bytes of the underlying buffer (>= the bytes of the current shape for tensors made by Reshape)
  int64_t rows() const { return n_dim() ? numel() / shape(-1) : 0; }  // product of all but the last dim
  DLDeviceType device_type() const { return view_.device.device_type; }
  int device_id() const { return view_.device.device_id; }
  DLDevice device_ctx() const { return view_.device; }
  DLDataType dtype() const { return view_.dtype; }
  bool on_gpu() const { return !is_null() && view_.device.device_type == kDLCUDA; }

  const void* raw() const { return is_null() ? nullptr : static_cast<const char*>(view_.data) + view_.byte_offset; }
  void* raw_mut() { return const_cast<void*>(raw()); }
  template <typename T> const T* data() const {
    TT_ENFORCE(!is_null() && SameType(view_.dtype, DataTypeTrait<T>::value()), "data type mismatch");
    return static_cast<const T*>(raw());
  }
  template <typename T> T* mutableData() { return const_cast<T*>(data<T>()); }

  // Makes this tensor hold `shape` of `dtype` on the device, keeping its storage when it owns enough
  // bytes on the same device (tensor.h:317-338 of the reference), else allocating by `name`.
  void* Reshape(DLDataType dtype, const std::vector<int64_t>& shape, DLDeviceType dev, int dev_id,
                const std::string& name = "Reshape");
  template <typename T>
  T* Reshape(const std::vector<int64_t>& shape, DLDeviceType dev, int dev_id, const std::string& name = "Reshape") {
    return static_cast<T*>(Reshape(DataTypeTrait<T>::value(), shape, dev, dev_id, name));
  }
  // Same storage seen under another shape with the same element count.
  void ViewAs(const std::vector<int64_t>& shape);

  // Non-owning view of sub-tensor n along the first axis.
  Tensor operator[](int64_t n) const;

  // Companion planes a layer may attach to a 16-bit activation it produced, for the next layer to use (they travel with
  // the tensor through moves, and are dropped when it is reshaped or exported):
  //   lo  : same shape and dtype, what rounding to the 16-bit type dropped (value = this + lo to 16 significant bits)
  //   f32 : same shape in fp32, the unrounded value (the residual stream of a bf16 model)
  const Tensor* lo() const;
  const Tensor* f32() const;
  const Tensor* q8() const;
  const Tensor* q8_scale() const;
  TensorExtras& NewExtras();
  void DropExtras() { extras_.reset(); }

 private:
  void Release();
  void MoveFrom(Tensor& o);
  DLManagedTensor* owned_ = nullptr;
  DLTensor view_{};      // what the accessors read; for an owning tensor a copy of owned_->dl_tensor
  bool is_view_ = false;
  std::vector<int64_t> view_shape_;  // backing store of view_.shape for views and re-shaped tensors
  std::shared_ptr<TensorExtras> extras_;
};

struct TensorExtras {
  Tensor lo{nullptr};
  Tensor f32{nullptr};
  // int8 models: the per-row symmetric int8 form of this activation and its row scales, written by the layer norm that
  // produced it so that the next int8 Linear does not quantise it again
  Tensor q8{nullptr};
  Tensor q8_scale{nullptr};
};
inline const Tensor* Tensor::lo() const { return extras_ && !extras_->lo.is_null() ? &extras_->lo : nullptr; }
inline const Tensor* Tensor::f32() const { return extras_ && !extras_->f32.is_null() ? &extras_->f32 : nullptr; }
inline const Tensor* Tensor::q8() const { return extras_ && !extras_->q8.is_null() ? &extras_->q8 : nullptr; }
inline const Tensor* Tensor::q8_scale() const { return extras_ && !extras_->q8_scale.is_null() ? &extras_->q8_scale : nullptr; }
inline TensorExtras& Tensor::NewExtras() {
  extras_ = std::make_shared<TensorExtras>();
  return *extras_;
}

// ---- module-level API of the reference kept for scripts that call it --------------------------------
void SetNumThreads(int n);  // host threads are not used by the device path; recorded only
void EnableGperf();
void DisableGperf();
namespace allocator {
void reset_allocator_schema(const std::string& name);  // "naive" | "model-aware"; both map to the device pool
void bert_opt_mem_allocate_api(int64_t batch_size, int64_t seq_len, int64_t num_head, int64_t hidden_size,
                               int64_t num_layer, const std::string& dev_str);
}  // namespace allocator

}  // namespace core
}  // namespace turbo_transformers
