// Test-infrastructure stand-in for the dlpack submodule (absent on this image): a current dlpack.h
// (its directory is put on the include path by build_ref.py as ORACLE_DLPACK_DIR) plus the
// pre-0.4 names the reference uses (DLContext, kDLGPU, the `ctx` field).
#pragma once
#include ORACLE_DLPACK_HEADER
typedef DLDevice DLContext;
#define kDLGPU kDLCUDA
#define ctx device
