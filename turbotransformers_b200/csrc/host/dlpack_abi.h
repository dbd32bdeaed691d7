// The DLPack in-memory tensor exchange ABI (struct layout of DLPack v0.x / the unversioned
// DLManagedTensor that torch.utils.dlpack produces and consumes), declared here so the host layer has no
// dependency on an external dlpack checkout.
#pragma once
#include <cstdint>

extern "C" {

typedef enum {
  kDLCPU = 1,
  kDLCUDA = 2,
  kDLCUDAHost = 3,
} DLDeviceType;

// The reference spells the CUDA device type kDLGPU; both names are accepted by this layer.
#define kDLGPU kDLCUDA

typedef struct {
  DLDeviceType device_type;
  int32_t device_id;
} DLDevice;

typedef enum {
  kDLInt = 0U,
  kDLUInt = 1U,
  kDLFloat = 2U,
  kDLOpaqueHandle = 3U,
  kDLBfloat = 4U,
} DLDataTypeCode;

typedef struct {
  uint8_t code;
  uint8_t bits;
  uint16_t lanes;
} DLDataType;

typedef struct {
  void* data;
  DLDevice device;
  int32_t ndim;
  DLDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
} DLTensor;

typedef struct DLManagedTensor {
  DLTensor dl_tensor;
  void* manager_ctx;
  void (*deleter)(struct DLManagedTensor* self);
} DLManagedTensor;

}  // extern "C"
