#include "core.h"

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>

namespace turbo_transformers {
namespace core {

// ---------------------------------------------------------------------------------------------------
// contexts
// ---------------------------------------------------------------------------------------------------
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_mu;
ttb_ctx* g_ctx[kMaxDevices] = {};
std::map<std::vector<int64_t>, CuSeqlensHandle> g_cu_cache[kMaxDevices];
int g_num_threads = 1;

struct Managed {
  DLManagedTensor dl;
  ttb_ctx* ctx = nullptr;  // null for host memory
  void* ptr = nullptr;
  size_t capacity = 0;
  std::vector<int64_t> shape;
};

void ManagedDeleter(DLManagedTensor* self) {
  auto* m = static_cast<Managed*>(self->manager_ctx);
  if (m->ptr) {
    if (m->ctx) ttb_free(m->ctx, m->ptr, "");
    else std::free(m->ptr);
  }
  delete m;
}

size_t ElemBytes(DLDataType dt) { return (size_t)(dt.bits / 8) * (dt.lanes ? dt.lanes : 1); }
}  // namespace

ttb_ctx* DeviceContext(int device_id) {
  TT_ENFORCE(device_id >= 0 && device_id < kMaxDevices, "device id %d out of range", device_id);
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_ctx[device_id]) {
    ttb_ctx* c = nullptr;
    int s = ttb_ctx_create(device_id, nullptr, &c);
    if (s != TTB_OK || !c) TT_THROW("cannot create a device context on GPU %d (status %d): is a CUDA device present?", device_id, s);
    g_ctx[device_id] = c;
  }
  return g_ctx[device_id];
}

void SetDeviceStream(int device_id, void* cuda_stream) {
  ttb_ctx* c = DeviceContext(device_id);
  if (ttb_ctx_stream(c) != cuda_stream) Check(ttb_ctx_set_stream(c, cuda_stream), c, "set_stream");
}

void Check(int status, ttb_ctx* ctx, const char* what) {
  if (status == TTB_OK) return;
  TT_THROW("%s failed with status %d: %s", what, status, ctx ? ttb_last_error(ctx) : "");
}

CuSeqlensHandle CuSeqlens(int device_id, const std::vector<int64_t>& seq_lens) {
  ttb_ctx* c = DeviceContext(device_id);
  std::vector<CuSeqlensHandle> evicted;  // released after the lock is dropped (the last release frees device memory)
  CuSeqlensHandle h;
  {
    std::lock_guard<std::mutex> g(g_mu);
    auto& cache = g_cu_cache[device_id];
    auto it = cache.find(seq_lens);
    if (it != cache.end()) return it->second;
    if (cache.size() >= 256) {  // arrays still held by a caller outlive this: only the cache's references go
      for (auto& kv : cache) evicted.push_back(std::move(kv.second));
      cache.clear();
    }
    void* p = nullptr;
    Check(ttb_alloc(c, (seq_lens.size() + 1) * sizeof(int32_t), "cu_seqlens", &p), c, "alloc cu_seqlens");
    h = CuSeqlensHandle(static_cast<const int32_t*>(p), [c](const int32_t* q) { ttb_free(c, const_cast<int32_t*>(q), "cu_seqlens"); });
    Check(ttb_build_cu_seqlens(c, seq_lens.data(), (int64_t)seq_lens.size(), static_cast<int32_t*>(p)), c, "build_cu_seqlens");
    cache[seq_lens] = h;
  }
  return h;
}

CuSeqlensHandle UniformCuSeqlens(int device_id, int64_t B, int64_t L) {
  return CuSeqlens(device_id, std::vector<int64_t>((size_t)B, L));
}

int ToTTBDtype(DLDataType dt) {
  if (dt.code == kDLFloat && dt.bits == 32) return TTB_F32;
  if (dt.code == kDLFloat && dt.bits == 16) return TTB_F16;
  if (dt.code == kDLBfloat && dt.bits == 16) return TTB_BF16;
  if (dt.code == kDLInt && dt.bits == 8) return TTB_I8;
  return -1;
}

// ---------------------------------------------------------------------------------------------------
// Tensor
// ---------------------------------------------------------------------------------------------------
DLManagedTensor* NewDLPackTensor(const std::vector<int64_t>& shape, DLDeviceType device, int device_id, DLDataType dtype,
                                 const std::string& name) {
  TT_ENFORCE(device == kDLCPU || device == kDLCUDA, "unsupported device type %d", (int)device);
  auto* m = new Managed();
  m->shape = shape;
  int64_t n = 1;
  for (int64_t d : shape) {
    TT_ENFORCE(d >= 0, "negative dimension in shape");
    n *= d;
  }
  const size_t bytes = (size_t)n * ElemBytes(dtype);
  m->capacity = bytes;
  if (bytes) {
    if (device == kDLCUDA) {
      m->ctx = DeviceContext(device_id);
      int s = ttb_alloc(m->ctx, bytes, name.c_str(), &m->ptr);
      if (s != TTB_OK) {
        std::string err = ttb_last_error(m->ctx);
        delete m;
        TT_THROW("allocation of %zu bytes for '%s' failed (status %d): %s", bytes, name.c_str(), s, err.c_str());
      }
    } else {
      m->ptr = std::aligned_alloc(64, (bytes + 63) / 64 * 64);
      if (!m->ptr) {
        delete m;
        TT_THROW("host allocation of %zu bytes failed", bytes);
      }
    }
  }
  m->dl.dl_tensor.data = m->ptr;
  m->dl.dl_tensor.device = {device, device_id};
  m->dl.dl_tensor.ndim = (int32_t)m->shape.size();
  m->dl.dl_tensor.dtype = dtype;
  m->dl.dl_tensor.shape = m->shape.data();
  m->dl.dl_tensor.strides = nullptr;
  m->dl.dl_tensor.byte_offset = 0;
  m->dl.manager_ctx = m;
  m->dl.deleter = ManagedDeleter;
  return &m->dl;
}

void Tensor::Release() {
  extras_.reset();
  if (owned_ && owned_->deleter) owned_->deleter(owned_);
  owned_ = nullptr;
  is_view_ = false;
  view_ = DLTensor{};
  view_shape_.clear();
}

void Tensor::MoveFrom(Tensor& o) {
  owned_ = o.owned_;
  view_ = o.view_;
  is_view_ = o.is_view_;
  const bool own_shape = !o.view_shape_.empty() && o.view_.shape == o.view_shape_.data();
  view_shape_ = std::move(o.view_shape_);
  if (own_shape) view_.shape = view_shape_.data();
  extras_ = std::move(o.extras_);
  o.owned_ = nullptr;
  o.is_view_ = false;
  o.view_ = DLTensor{};
  o.view_shape_.clear();
}

DLManagedTensor* Tensor::ToDLPack() {
  TT_ENFORCE(owned_ != nullptr, "only a tensor that owns its storage can be exported through DLPack");
  DLManagedTensor* t = owned_;
  owned_ = nullptr;
  Release();
  return t;
}

int64_t Tensor::shape(int pos) const {
  TT_ENFORCE(!is_null(), "shape() of a null tensor");
  if (pos < 0) pos += view_.ndim;
  TT_ENFORCE(pos >= 0 && pos < view_.ndim, "shape index %d out of range for %d dims", pos, view_.ndim);
  return view_.shape[pos];
}

int64_t Tensor::numel() const {
  if (is_null()) return 0;
  int64_t n = 1;
  for (int i = 0; i < view_.ndim; ++i) n *= view_.shape[i];
  return n;
}

void* Tensor::Reshape(DLDataType dtype, const std::vector<int64_t>& shape, DLDeviceType dev, int dev_id, const std::string& name) {
  int64_t n = 1;
  for (int64_t d : shape) n *= d;
  const size_t need = (size_t)n * ElemBytes(dtype);
  extras_.reset();  // the contents are about to be replaced
  if (owned_ && owned_->deleter == ManagedDeleter) {
    auto* m = static_cast<Managed*>(owned_->manager_ctx);
    if (m->capacity >= need && view_.device.device_type == dev && view_.device.device_id == dev_id) {
      m->shape = shape;
      owned_->dl_tensor.shape = m->shape.data();
      owned_->dl_tensor.ndim = (int32_t)shape.size();
      owned_->dl_tensor.dtype = dtype;
      view_ = owned_->dl_tensor;
      return raw_mut();
    }
  }
  Release();
  owned_ = NewDLPackTensor(shape, dev, dev_id, dtype, name);
  view_ = owned_->dl_tensor;
  return raw_mut();
}

size_t Tensor::capacity_bytes() const {
  if (is_null()) return 0;
  if (owned_ && owned_->deleter == ManagedDeleter) return static_cast<Managed*>(owned_->manager_ctx)->capacity;
  return (size_t)numel() * ElemBytes(view_.dtype);
}

void Tensor::ViewAs(const std::vector<int64_t>& shape) {
  int64_t n = 1;
  for (int64_t d : shape) n *= d;
  TT_ENFORCE_EQ(n, numel(), "ViewAs must keep the element count");
  if (owned_ && owned_->deleter == ManagedDeleter) {
    auto* m = static_cast<Managed*>(owned_->manager_ctx);
    m->shape = shape;
    owned_->dl_tensor.shape = m->shape.data();
    owned_->dl_tensor.ndim = (int32_t)shape.size();
    view_ = owned_->dl_tensor;
    return;
  }
  view_shape_ = shape;
  view_.shape = view_shape_.data();
  view_.ndim = (int32_t)shape.size();
}

Tensor Tensor::operator[](int64_t n) const {
  TT_ENFORCE(!is_null() && view_.ndim >= 2, "operator[] needs at least two dims");
  TT_ENFORCE(n >= 0 && n < view_.shape[0], "operator[] index out of range");
  Tensor t(nullptr);
  t.is_view_ = true;
  t.view_ = view_;
  t.view_shape_.assign(view_.shape + 1, view_.shape + view_.ndim);
  t.view_.shape = t.view_shape_.data();
  t.view_.ndim = view_.ndim - 1;
  int64_t inner = 1;
  for (int64_t d : t.view_shape_) inner *= d;
  t.view_.byte_offset = view_.byte_offset + (uint64_t)(n * inner) * ElemBytes(view_.dtype);
  return t;
}

// ---------------------------------------------------------------------------------------------------
// precision switches
// ---------------------------------------------------------------------------------------------------
namespace {
int g_precise_bf16 = -1, g_fp32_tc = -1;  // -1: not decided yet (environment)
}
bool PreciseBF16() {
  if (g_precise_bf16 < 0) {
    const char* e = std::getenv("TTB_BF16_PRECISE");
    g_precise_bf16 = (e && e[0] == '0') ? 0 : 1;
  }
  return g_precise_bf16 != 0;
}
void SetPreciseBF16(bool on) { g_precise_bf16 = on ? 1 : 0; }
bool Fp32TensorCores() {
  if (g_fp32_tc < 0) {
    const char* e = std::getenv("TTB_FP32_GEMM");
    g_fp32_tc = (e && std::string(e) == "simt") ? 0 : 1;
  }
  return g_fp32_tc != 0;
}
void SetFp32TensorCores(bool on) { g_fp32_tc = on ? 1 : 0; }

// ---------------------------------------------------------------------------------------------------
// module-level API
// ---------------------------------------------------------------------------------------------------
void SetNumThreads(int n) { g_num_threads = n; }
void EnableGperf() {}
void DisableGperf() {}

namespace allocator {
void reset_allocator_schema(const std::string& name) {
  TT_ENFORCE(name == "naive" || name == "model-aware", "unknown allocator schema '%s'", name.c_str());
}
void bert_opt_mem_allocate_api(int64_t batch_size, int64_t seq_len, int64_t num_head, int64_t hidden_size,
                               int64_t num_layer, const std::string& dev_str) {
  if (dev_str != "GPU") return;  // host activations are not used by this runtime
  ttb_ctx* c = DeviceContext(0);
  size_t arena = 0;
  Check(ttb_plan_activations(c, batch_size, batch_size * seq_len, num_head, hidden_size, 4 * hidden_size, num_layer, TTB_F32, &arena), c,
        "plan_activations");
}
}  // namespace allocator

}  // namespace core
}  // namespace turbo_transformers
