// pybind11 module `turbo_transformers_cxx`: the same module name, class names, constructor argument
// order and __call__ signatures as the reference's turbo_transformers/python/pybind.cpp:141-371, bound
// to the layer classes in layers.h. Extra methods (quantize_int8, set_* switches, packed helpers,
// set_stream) are additions; nothing the reference exported for this path is missing.
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>

#include "bert_model.h"
#include "layers.h"
#include "npz.h"

namespace py = pybind11;
using namespace turbo_transformers;
using core::Tensor;

namespace {

void CapsuleDestructor(PyObject* capsule) {
  // A consumer renames the capsule when it takes the tensor; an unconsumed one still owns it.
  if (PyCapsule_IsValid(capsule, "dltensor")) {
    auto* t = static_cast<DLManagedTensor*>(PyCapsule_GetPointer(capsule, "dltensor"));
    if (t && t->deleter) t->deleter(t);
  }
}

template <typename T>
Tensor* NumpyToTensor(py::array_t<T, py::array::c_style | py::array::forcecast> arr, const std::string& dev) {
  std::vector<int64_t> shape(arr.ndim());
  for (py::ssize_t i = 0; i < arr.ndim(); ++i) shape[i] = arr.shape(i);
  const bool gpu = dev == "GPU";
  TT_ENFORCE(gpu || dev == "CPU", "device must be \"CPU\" or \"GPU\"");
  auto* t = new Tensor(core::NewDLPackTensor(shape, gpu ? kDLCUDA : kDLCPU, 0, core::DataTypeTrait<T>::value(), "nparray2tensor"));
  const size_t bytes = (size_t)arr.size() * sizeof(T);
  if (gpu) {
    ttb_ctx* c = core::DeviceContext(0);
    core::Check(ttb_memcpy_h2d(c, t->raw_mut(), arr.data(), bytes), c, "nparray2tensor");
  } else if (bytes) {
    std::memcpy(t->raw_mut(), arr.data(), bytes);
  }
  return t;
}

template <typename T> py::array_t<T> TensorToNumpy(const Tensor& t) {
  TT_ENFORCE(!t.is_null(), "tensor is null");
  TT_ENFORCE(core::SameType(t.dtype(), core::DataTypeTrait<T>::value()), "tensor dtype does not match the requested numpy dtype");
  std::vector<py::ssize_t> shape(t.n_dim());
  for (size_t i = 0; i < shape.size(); ++i) shape[i] = t.shape((int)i);
  py::array_t<T> out(shape);
  const size_t bytes = (size_t)t.numel() * sizeof(T);
  if (t.on_gpu()) {
    ttb_ctx* c = core::DeviceContext(t.device_id());
    core::Check(ttb_memcpy_d2h(c, out.mutable_data(), t.raw(), bytes), c, "tensor2nparray");
  } else if (bytes) {
    std::memcpy(out.mutable_data(), t.raw(), bytes);
  }
  return out;
}

std::string DtypeName(const Tensor& t) {
  if (t.is_null()) return "null";
  DLDataType d = t.dtype();
  if (d.code == kDLFloat) return "float" + std::to_string(d.bits);
  if (d.code == kDLBfloat) return "bfloat16";
  if (d.code == kDLInt) return "int" + std::to_string(d.bits);
  return "unknown";
}

}  // namespace

PYBIND11_MODULE(turbo_transformers_cxx, m) {
  py::register_exception<core::details::EnforceNotMet>(m, "EnforceNotMet", PyExc_RuntimeError);

  auto config = m.def_submodule("config", "compile configuration");
  config.def("is_compiled_with_cuda", [] { return true; });
  config.def("get_blas_provider", [] { return std::string("tcgen05"); });

  m.def("nparray2tensor", &NumpyToTensor<float>, py::return_value_policy::take_ownership, "Convert Numpy to Tensor.");
  m.def("nparray2tensor", &NumpyToTensor<int64_t>, py::return_value_policy::take_ownership, "Convert Numpy to Tensor.");
  m.def("tensor2nparrayf", &TensorToNumpy<float>, "Convert Tensor to Numpy, float data only.");
  m.def("tensor2nparrayl", &TensorToNumpy<int64_t>, "Convert Tensor to Numpy, int64 data only.");
  m.def("set_stderr_verbose_level", [](int) {});
  m.def("enable_perf", &core::EnableGperf);
  m.def("disable_perf", &core::DisableGperf);
  m.def("set_num_threads", &core::SetNumThreads);
  m.def("bert_opt_mem_allocate_api", &core::allocator::bert_opt_mem_allocate_api);
  m.def("reset_allocator_schema", &core::allocator::reset_allocator_schema);
  // additions
  m.def("set_stream", [](int device, uintptr_t stream) { core::SetDeviceStream(device, reinterpret_cast<void*>(stream)); },
        "Run this device's kernels on the given cudaStream_t (0 = the legacy default stream).");
  m.def("synchronize", [](int device) { ttb_ctx* c = core::DeviceContext(device); core::Check(ttb_ctx_sync(c), c, "synchronize"); });
  m.def("device_status", [](int device) { return ttb_device_status(core::DeviceContext(device)); },
        "Synchronise and return the device-side status word (0 = OK), clearing it.");
  m.def("launch_count", [](int device) { return ttb_launch_count(core::DeviceContext(device)); });
  m.def("arena_begin", [](int device, size_t bytes) { ttb_ctx* c = core::DeviceContext(device); core::Check(ttb_arena_begin(c, bytes), c, "arena_begin"); },
        "Serve every allocation from one reserved buffer at fixed offsets until arena_end (for CUDA-graph capture of a forward pass).");
  m.def("arena_end", [](int device) {
    ttb_ctx* c = core::DeviceContext(device);
    size_t used = 0;
    void* arena = nullptr;
    core::Check(ttb_arena_end(c, &used, &arena), c, "arena_end");
    return std::make_pair(used, reinterpret_cast<uintptr_t>(arena));
  }, "End arena mode; returns (bytes used, arena handle). The buffer stays reserved until arena_release(device, handle).");
  m.def("arena_release", [](int device, uintptr_t arena) {
    ttb_ctx* c = core::DeviceContext(device);
    core::Check(ttb_arena_release(c, reinterpret_cast<void*>(arena)), c, "arena_release");
  });
  m.def("set_bf16_precise", [](bool on) { core::SetPreciseBF16(on); },
        "bf16 models: keep an fp32 residual stream and hi + lo activation planes between layers (default on).");
  m.def("bf16_precise", []() { return core::PreciseBF16(); });
  m.def("set_fp32_tensor_cores", [](bool on) { core::SetFp32TensorCores(on); },
        "fp32 models: run Linears on the tensor cores as three tf32 products (default on); off = exact-order CUDA-core GEMM.");
  m.def("fp32_tensor_cores", []() { return core::Fp32TensorCores(); });
  m.def("bytes_allocated_total", [](int device) {
    ttb_ctx* c = core::DeviceContext(device);
    uint64_t b = 0;
    core::Check(ttb_bytes_allocated_total(c, &b), c, "bytes_allocated_total");
    return b;
  });
  m.def("pool_stats", [](int device) {
    size_t in_use = 0, high = 0;
    uint64_t n = 0;
    ttb_pool_stats(core::DeviceContext(device), &in_use, &high, &n);
    return py::make_tuple(in_use, high, n);
  });
  m.def("plan_activations", [](int device, int64_t batch, int64_t tokens, int64_t heads, int64_t hidden, int64_t ffn, int64_t layers,
                               int dtype) {
    size_t arena = 0;
    ttb_ctx* c = core::DeviceContext(device);
    core::Check(ttb_plan_activations(c, batch, tokens, heads, hidden, ffn, layers, dtype, &arena), c, "plan_activations");
    return arena;
  });

  py::class_<Tensor>(m, "Tensor")
      .def_static("from_dlpack",
                  [](py::capsule capsule) -> std::unique_ptr<Tensor> {
                    auto* t = static_cast<DLManagedTensor*>(capsule);
                    PyCapsule_SetName(capsule.ptr(), "used_tensor");
                    return std::make_unique<Tensor>(t);
                  })
      .def("to_dlpack",
           [](Tensor& t) -> py::capsule { return py::capsule(t.ToDLPack(), "dltensor", CapsuleDestructor); })
      .def("n_dim", &Tensor::n_dim)
      .def("shape", &Tensor::shape)
      .def("is_null", &Tensor::is_null)
      .def("dtype", &DtypeName)
      .def("numel", &Tensor::numel)
      .def_static("create_empty", [] { return Tensor(nullptr); });

  py::class_<layers::BERTEmbedding>(m, "BERTEmbedding")
      .def(py::init([](Tensor& word, Tensor& position, Tensor& token_type, Tensor& ln_w, Tensor& ln_b) {
        return new layers::BERTEmbedding(std::move(word), std::move(position), std::move(token_type), std::move(ln_w), std::move(ln_b));
      }))
      .def("__call__", &layers::BERTEmbedding::operator())
      .def("packed", [](const layers::BERTEmbedding& self, const Tensor& ids, const std::vector<int64_t>& lens, Tensor* out,
                        const Tensor* position_ids, const Tensor* token_type_ids) {
        const Tensor none(nullptr);
        self.Packed(ids, lens, out, position_ids ? *position_ids : none, token_type_ids ? *token_type_ids : none);
      }, py::arg("input_ids"), py::arg("seq_lens"), py::arg("output"), py::arg("position_ids") = nullptr, py::arg("token_type_ids") = nullptr);

  py::class_<layers::BertAttention>(m, "BertAttention")
      .def(py::init([](Tensor& qkv_weight, Tensor& qkv_bias, Tensor& dense_weight, Tensor& dense_bias, Tensor& ln_w, Tensor& ln_b,
                       int num_attention_heads) {
        return new layers::BertAttention(std::move(qkv_weight), std::move(qkv_bias), std::move(dense_weight), std::move(dense_bias),
                                         std::move(ln_w), std::move(ln_b), num_attention_heads);
      }))
      .def("__call__", &layers::BertAttention::operator())
      .def("quantize_int8", [](layers::BertAttention& s) { s.QuantizeInt8(); });

  py::class_<layers::MultiHeadedAttention>(m, "MultiHeadedAttention")
      .def(py::init([](Tensor& kw, Tensor& kb, Tensor& vw, Tensor& vb, Tensor& qw, Tensor& qb, Tensor& dw, Tensor& db, Tensor& qkvw,
                       Tensor& qkvb, int heads) {
        return new layers::MultiHeadedAttention(std::move(kw), std::move(kb), std::move(vw), std::move(vb), std::move(qw), std::move(qb),
                                                std::move(dw), std::move(db), std::move(qkvw), std::move(qkvb), heads);
      }))
      .def(py::init([](Tensor& kw, Tensor& kb, Tensor& vw, Tensor& vb, Tensor& qw, Tensor& qb, Tensor& dw, Tensor& db, Tensor& qkvw,
                       Tensor& qkvb, Tensor& ln_g, Tensor& ln_b, int heads) {
        return new layers::MultiHeadedAttention(std::move(kw), std::move(kb), std::move(vw), std::move(vb), std::move(qw), std::move(qb),
                                                std::move(dw), std::move(db), std::move(qkvw), std::move(qkvb), std::move(ln_g),
                                                std::move(ln_b), heads);
      }))
      .def("__call__", &layers::MultiHeadedAttention::operator())
      .def("set_pre_layernorm_eps", &layers::MultiHeadedAttention::set_pre_layernorm_eps)
      .def("set_causal", &layers::MultiHeadedAttention::set_causal)
      .def("quantize_int8", &layers::MultiHeadedAttention::QuantizeInt8);

  py::class_<layers::MultiHeadedAttentionSmartBatch>(m, "MultiHeadedAttentionSmartBatch")
      .def(py::init([](Tensor& kw, Tensor& kb, Tensor& vw, Tensor& vb, Tensor& qw, Tensor& qb, Tensor& dw, Tensor& db, Tensor& qkvw,
                       Tensor& qkvb, int heads) {
        return new layers::MultiHeadedAttentionSmartBatch(std::move(kw), std::move(kb), std::move(vw), std::move(vb), std::move(qw),
                                                          std::move(qb), std::move(dw), std::move(db), std::move(qkvw), std::move(qkvb),
                                                          heads);
      }))
      .def(py::init([](Tensor& kw, Tensor& kb, Tensor& vw, Tensor& vb, Tensor& qw, Tensor& qb, Tensor& dw, Tensor& db, Tensor& qkvw,
                       Tensor& qkvb, Tensor& ln_g, Tensor& ln_b, int heads) {
        return new layers::MultiHeadedAttentionSmartBatch(std::move(kw), std::move(kb), std::move(vw), std::move(vb), std::move(qw),
                                                          std::move(qb), std::move(dw), std::move(db), std::move(qkvw), std::move(qkvb),
                                                          std::move(ln_g), std::move(ln_b), heads);
      }))
      .def("__call__", &layers::MultiHeadedAttentionSmartBatch::operator())
      .def("quantize_int8", [](layers::MultiHeadedAttentionSmartBatch& s) { s.QuantizeInt8(); });

  py::class_<layers::BertIntermediate>(m, "BertIntermediate")
      .def(py::init([](Tensor& w, Tensor& b) { return new layers::BertIntermediate(std::move(w), std::move(b)); }))
      .def("__call__", &layers::BertIntermediate::operator())
      .def("quantize_int8", &layers::BertIntermediate::QuantizeInt8, py::arg("mode") = 1);

  py::class_<layers::BertOutput>(m, "BertOutput")
      .def(py::init([](Tensor& w, Tensor& b, Tensor& ln_w, Tensor& ln_b) {
        return new layers::BertOutput(std::move(w), std::move(b), std::move(ln_w), std::move(ln_b));
      }))
      .def("__call__", &layers::BertOutput::operator())
      .def("quantize_int8", &layers::BertOutput::QuantizeInt8, py::arg("mode") = 1);

  py::class_<layers::SequencePool>(m, "SequencePool")
      .def(py::init([](const std::string& pool_type) { return new layers::SequencePool(pool_type); }))
      .def("__call__", &layers::SequencePool::operator())
      .def("packed", &layers::SequencePool::Packed);

  py::class_<layers::BertPooler>(m, "BertPooler")
      .def(py::init([](Tensor& w, Tensor& b) { return new layers::BertPooler(std::move(w), std::move(b)); }))
      .def("__call__", &layers::BertPooler::operator());

  // ---- the Python-free model of the C++ API (example/cpp/bert_model.cpp of the reference), reachable from Python for tests
  m.def("npz_load", [](const std::string& filename) {
    py::dict d;
    for (auto& kv : loaders::npz_load(filename)) {
      d[py::str(kv.first)] = py::make_tuple(kv.second.descr, kv.second.shape,
                                            py::bytes(reinterpret_cast<const char*>(kv.second.bytes.data()), kv.second.bytes.size()));
    }
    return d;
  }, "Read an .npz archive with the C++ reader: {name: (dtype string, shape, raw bytes)}.");
  py::class_<BertModel>(m, "NpzBertModel")
      .def(py::init([](const std::string& filename, size_t n_layers, int64_t n_heads, const std::string& dtype, int device_id) {
             return new BertModel(filename, kDLCUDA, n_layers, n_heads, dtype, device_id);
           }),
           py::arg("filename"), py::arg("n_layers"), py::arg("n_heads"), py::arg("dtype") = "float32", py::arg("device_id") = 0)
      .def("__call__",
           [](const BertModel& self, const std::vector<std::vector<int64_t>>& inputs, const std::vector<std::vector<int64_t>>& position_ids,
              const std::vector<std::vector<int64_t>>& segment_ids, const std::string& pooling, bool use_pooler) {
             PoolType p = PoolType::kFirst;
             if (pooling == "Max") p = PoolType::kMax;
             else if (pooling == "Mean") p = PoolType::kMean;
             else if (pooling == "Last") p = PoolType::kLast;
             else if (pooling != "First") TT_THROW("The input pool type (%s) is not supported.", pooling.c_str());
             return self(inputs, position_ids, segment_ids, p, use_pooler);
           },
           py::arg("inputs"), py::arg("position_ids") = std::vector<std::vector<int64_t>>(),
           py::arg("segment_ids") = std::vector<std::vector<int64_t>>(), py::arg("pooling") = "First", py::arg("use_pooler") = false)
      .def_property_readonly("hidden_size", &BertModel::hidden_size);

  py::class_<layers::PrepareBertMasks>(m, "PrepareBertMasks").def(py::init()).def("__call__", &layers::PrepareBertMasks::operator());

  py::class_<layers::DistrillFFN>(m, "DistrillFFN")
      .def(py::init([](Tensor& w1, Tensor& b1, Tensor& w2, Tensor& b2, Tensor& ln_w, Tensor& ln_b) {
        return new layers::DistrillFFN(std::move(w1), std::move(b1), std::move(w2), std::move(b2), std::move(ln_w), std::move(ln_b));
      }))
      .def("__call__", &layers::DistrillFFN::operator(), py::arg("input_tensor"), py::arg("output"), py::arg("is_trans_weight") = true);

  py::class_<layers::AlbertLayer>(m, "AlbertLayer")
      .def(py::init([](Tensor& w1, Tensor& b1, Tensor& w2, Tensor& b2, Tensor& ln_w, Tensor& ln_b) {
        return new layers::AlbertLayer(std::move(w1), std::move(b1), std::move(w2), std::move(b2), std::move(ln_w), std::move(ln_b));
      }))
      .def("__call__", &layers::AlbertLayer::operator());

  py::class_<layers::PositionwiseFeedForward>(m, "PositionwiseFeedForward")
      .def(py::init([](Tensor& w1, Tensor& b1, Tensor& w2, Tensor& b2, Tensor& ln_w, Tensor& ln_b) {
        return new layers::PositionwiseFeedForward(std::move(w1), std::move(b1), std::move(w2), std::move(b2), std::move(ln_w),
                                                   std::move(ln_b));
      }))
      .def("__call__", &layers::PositionwiseFeedForward::operator())
      .def("set_activation", &layers::PositionwiseFeedForward::set_activation)
      .def("set_layernorm_eps", &layers::PositionwiseFeedForward::set_layernorm_eps);

  py::class_<layers::FusedAddBiasGELU>(m, "FusedAddBiasGELU")
      .def(py::init([](Tensor& bias) { return new layers::FusedAddBiasGELU(std::move(bias)); }))
      .def("__call__", &layers::FusedAddBiasGELU::operator());

  py::class_<layers::FusedAddBiasLayerNorm>(m, "FusedAddBiasLayerNorm")
      .def(py::init([](Tensor& bias, Tensor& ln_w, Tensor& ln_b) {
        return new layers::FusedAddBiasLayerNorm(std::move(bias), std::move(ln_w), std::move(ln_b));
      }))
      .def("__call__", &layers::FusedAddBiasLayerNorm::operator());

  py::class_<layers::LayerNorm>(m, "LayerNorm")
      .def(py::init([](Tensor& g, Tensor& b, float eps) { return new layers::LayerNorm(std::move(g), std::move(b), eps); }))
      .def("__call__", &layers::LayerNorm::operator());

  py::class_<layers::TokenPositionEmbedding>(m, "TokenPositionEmbedding")
      .def(py::init([](Tensor& tok, Tensor& pos) { return new layers::TokenPositionEmbedding(std::move(tok), std::move(pos)); }))
      .def("__call__", &layers::TokenPositionEmbedding::operator(), py::arg("input_ids"), py::arg("output"), py::arg("position_offset") = 0);

  py::class_<layers::Linear>(m, "Linear")
      .def(py::init([](Tensor& w, Tensor& b, bool is_trans_weight) { return new layers::Linear(std::move(w), std::move(b), is_trans_weight); }))
      .def("__call__", &layers::Linear::operator())
      .def("padded", &layers::Linear::Padded,
           "The product with the output's last dimension rounded up to a multiple of 8 (columns beyond width() are undefined).")
      .def("width", &layers::Linear::Width)
      .def("padded_width", &layers::Linear::PaddedWidth);
}
