// `.npz` weight archives for the C++ API: the container the reference's converter writes
// (tools/convert_huggingface_bert_pytorch_to_npz.py:23-74) and its loader reads (turbo_transformers/loaders/npz_load.h:23-75,
// through the cnpy library there). This reader has no dependency beyond zlib: a `.npz` is a zip archive of `.npy` members,
// stored (numpy.savez) or deflated (numpy.savez_compressed), with zip64 fields as numpy writes them.
//
// NPZMapView / NPZLoader keep the reference's names and methods (Sub, IsExist, operator[], LoadFloat); the loader places
// tensors on a CUDA device in the model's dtype (fp32 members are converted on the device for fp16 / bf16 models).
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <utility>
#include <vector>

#include "core.h"

namespace turbo_transformers {
namespace loaders {

struct NpyArray {
  std::string descr;           // numpy dtype string, e.g. "<f4"
  bool fortran_order = false;
  std::vector<int64_t> shape;
  size_t word_size = 0;
  std::vector<uint8_t> bytes;  // C-order payload
  size_t num_vals() const;
  template <typename T> const T* data() const { return reinterpret_cast<const T*>(bytes.data()); }
};
using npz_t = std::map<std::string, NpyArray>;

// Reads every member of the archive. Throws EnforceNotMet on a malformed file or an unsupported member.
npz_t npz_load(const std::string& filename);
// One `.npy` image (the payload of a zip member, or a whole `.npy` file).
NpyArray npy_parse(const uint8_t* data, size_t size, const std::string& what);

class NPZMapView {
 public:
  NPZMapView(std::string prefix, npz_t* npz) : prefix_(std::move(prefix)), npz_(npz) {}
  NpyArray& operator[](const std::string& key);
  NPZMapView Sub(const std::string& subview) { return NPZMapView(prefix_ + subview + ".", npz_); }
  bool IsExist(const std::string& subprefix) const;

 private:
  std::string prefix_;
  npz_t* npz_;
};

class NPZLoader {
 public:
  // dtype: the model's parameter type (fp32, fp16 or bf16); members must be '<f4' or '<f2'.
  NPZLoader(NPZMapView view, DLDeviceType device, int device_id = 0, DLDataType dtype = {kDLFloat, 32, 1})
      : view_(std::move(view)), device_(device), device_id_(device_id), dtype_(dtype) {}
  core::Tensor LoadFloat(const std::string& name);
  core::Tensor operator[](const std::string& name) { return LoadFloat(name); }

 private:
  NPZMapView view_;
  DLDeviceType device_;
  int device_id_;
  DLDataType dtype_;
};

}  // namespace loaders
}  // namespace turbo_transformers
