// Host-side helpers shared by the ahead-of-time library and the per-config libraries the tuner
// compiles: status codes, last-error text, TMA tensor-map encoding through the driver entry point
// (no link-time dependency on libcuda), device status read-back.
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "ptx.cuh"

namespace ab200 {

// Return codes of every C-ABI entry point.
enum : int {
  kOk = 0,
  kErrInvalidArgument = 1,  // null pointer, non-positive size, misaligned pointer, bad dtype
  kErrUnsupported = 2,      // head dims / config not built into this library
  kErrCuda = 3,             // a CUDA runtime / driver call failed (text in last_error)
  kErrDevice = 4,           // a kernel reported a non-zero device status (bounded wait expired)
};

inline char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }();
  return fn;
}

// Rank-3 map over a dense [d2][d1][d0] tensor of 16-bit elements (d0 contiguous), boxes of
// box0 x box1 x 1 elements, 128-byte swizzle (box0 * 2 bytes must be 128).
inline int make_tmap_3d(CUtensorMap* m, const void* base, bool bf16, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint32_t box0, uint32_t box1) {
  auto enc = tensor_map_encoder();
  if (!enc) return fail(kErrCuda, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * 2, d0 * d1 * 2};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   box0 * 2 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(kErrCuda, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return kOk;
}

inline int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(kErrCuda, "%s: %s", what, cudaGetErrorString(e));
  return kOk;
}

// Synchronises the device and returns the sticky device status word (0 = ok); clears it when asked.
inline int read_device_status(int clear, int* detail) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(kErrCuda, "cudaDeviceSynchronize: %s", cudaGetErrorString(e)), -1;
  int st = 0, det = 0;
  if (cudaMemcpyFromSymbol(&st, g_device_status, sizeof(int)) != cudaSuccess ||
      cudaMemcpyFromSymbol(&det, g_device_status_detail, sizeof(int)) != cudaSuccess) {
    fail(kErrCuda, "cudaMemcpyFromSymbol(device status): %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  if (detail) *detail = det;
  if (clear && st != 0) {
    int zero = 0;
    cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    cudaMemcpyToSymbol(g_device_status_detail, &zero, sizeof(int));
  }
  if (st != 0) fail(kErrDevice, "device status %d (tag %d, block %d)", st, det >> 16, det & 0xffff);
  return st;
}

// The tensor maps are encoded through the driver API, which needs a context current on the calling
// thread; threads that have only ever been handed tensors (e.g. an autograd worker) may not have one yet.
// Checks that `ptr` is device memory of the thread's current device and binds that device's primary context.
inline int bind_device_of(const void* ptr, const char* what) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, ptr) != cudaSuccess) {
    cudaError_t e = cudaGetLastError();
    return fail(kErrCuda, "%s: cudaPointerGetAttributes: %s", what, cudaGetErrorString(e));
  }
  if (at.type != cudaMemoryTypeDevice && at.type != cudaMemoryTypeManaged)
    return fail(kErrInvalidArgument, "%s: tensor pointer is not device memory", what);
  int cur = -1;
  cudaGetDevice(&cur);
  if (at.type == cudaMemoryTypeDevice && cur != at.device)
    return fail(kErrInvalidArgument, "%s: tensors live on device %d but the calling thread's current device is %d", what,
                at.device, cur);
  cudaError_t e = cudaFree(nullptr);  // binds the primary context to this thread if it is not yet
  if (e != cudaSuccess) return fail(kErrCuda, "%s: context initialisation: %s", what, cudaGetErrorString(e));
  return kOk;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

}  // namespace ab200
