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

#include <mutex>

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

// Set (per thread) for the duration of an entry point that promised its caller to allocate nothing: the helpers below
// that would otherwise create something on their first use on a device (the pinned status mirror, the context-binding
// cudaFree(nullptr)) skip that step while it is set. Every other entry point leaves it clear.
inline bool& no_alloc_scope_flag() {
  static thread_local bool flag = false;
  return flag;
}
struct NoAllocScope {
  bool prev;
  NoAllocScope() : prev(no_alloc_scope_flag()) { no_alloc_scope_flag() = true; }
  ~NoAllocScope() { no_alloc_scope_flag() = prev; }
};

// Host-visible mirror of the device status words of THIS library on the calling thread's current device: four ints in
// mapped pinned host memory ([0] status, [1] detail, [2] numeric flag) that report_timeout() / report_saturation() write
// next to the device-side words.
// Created on the first call per device (a few bytes of pinned host memory that live until the process exits; one
// synchronous copy of the pointer into the device symbol). Returns nullptr, with the error text set, if that fails.
// Internal linkage on purpose: the table pairs with THIS library's g_status_mirror symbol, and the local statics of an
// inline function would be shared by every library of the process that contains the same function.
static volatile int* status_mirror() {
  constexpr int kMaxDevices = 64;
  static volatile int* table[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(kErrCuda, "status mirror: no usable current device");
    return nullptr;
  }
  if (table[dev] != nullptr) return table[dev];
  if (no_alloc_scope_flag()) return nullptr;  // not created yet, and the caller may not allocate: do without it
  std::lock_guard<std::mutex> lock(mu);
  if (table[dev] != nullptr) return table[dev];
  int* host = nullptr;
  int* devptr = nullptr;
  cudaError_t e = cudaHostAlloc(reinterpret_cast<void**>(&host), 4 * sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable);
  if (e == cudaSuccess) {
    host[0] = host[1] = host[2] = host[3] = 0;
    e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&devptr), host, 0);
  }
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_status_mirror, &devptr, sizeof(devptr));
  if (e != cudaSuccess) {
    fail(kErrCuda, "status mirror set-up: %s", cudaGetErrorString(e));
    (void)cudaGetLastError();
    return nullptr;
  }
  table[dev] = host;
  return host;
}

// Called by every launcher before it launches: refuses to run while the sticky status word of an earlier kernel is
// still set (every bounded wait would give up at once and the outputs would be garbage). No synchronisation: the
// word is read from the host-mapped mirror.
static int check_prior_status(const char* what) {
  volatile int* m = status_mirror();
  if (m == nullptr) return no_alloc_scope_flag() ? kOk : kErrCuda;
  if (m[0] != 0) {
    const int det = m[1];
    return fail(kErrDevice,
                "%s: an earlier kernel of this library gave up on a bounded wait (status %d, tag %d, block %d); results "
                "since then are invalid. Read and clear the status (device_status(1)) before launching again",
                what, m[0], det >> 16, det & 0xffff);
  }
  if (m[2] != 0)
    return fail(kErrDevice,
                "%s: an earlier RetNet forward of this library clamped unnormalised scores to the fp16 range (status 2); its "
                "output is not trustworthy. Use bf16 or smaller inputs; read and clear the status (device_status(1)) before "
                "launching again", what);
  return kOk;
}

// Synchronises the device and returns the sticky device status word (0 = ok); clears it when asked.
inline int read_device_status(int clear, int* detail) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(kErrCuda, "cudaDeviceSynchronize: %s", cudaGetErrorString(e)), -1;
  int st = 0, det = 0, num = 0;
  if (cudaMemcpyFromSymbol(&st, g_device_status, sizeof(int)) != cudaSuccess ||
      cudaMemcpyFromSymbol(&det, g_device_status_detail, sizeof(int)) != cudaSuccess ||
      cudaMemcpyFromSymbol(&num, g_numeric_status, sizeof(int)) != cudaSuccess) {
    fail(kErrCuda, "cudaMemcpyFromSymbol(device status): %s", cudaGetErrorString(cudaGetLastError()));
    return -1;
  }
  if (detail) *detail = det;
  if (clear && (st != 0 || num != 0)) {
    int zero = 0;
    cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
    cudaMemcpyToSymbol(g_device_status_detail, &zero, sizeof(int));
    cudaMemcpyToSymbol(g_numeric_status, &zero, sizeof(int));
    volatile int* m = status_mirror();
    if (m != nullptr) m[0] = m[1] = m[2] = 0;
  }
  if (st != 0) {
    fail(kErrDevice, "device status %d (tag %d, block %d)", st, det >> 16, det & 0xffff);
    return st;
  }
  if (num != 0) {
    fail(kErrDevice, "device status %d: a RetNet forward clamped unnormalised scores to the fp16 range (|q k^T * scale * mask| "
                     "above 65504); its output is not trustworthy. Use bf16 or smaller inputs", (int)kStatusSaturated);
    return kStatusSaturated;
  }
  return 0;
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
  if (no_alloc_scope_flag()) return kOk;  // the entry point has bound the context itself (cudaGetSymbolAddress)
  cudaError_t e = cudaFree(nullptr);  // binds the primary context to this thread if it is not yet
  if (e != cudaSuccess) return fail(kErrCuda, "%s: context initialisation: %s", what, cudaGetErrorString(e));
  return kOk;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

}  // namespace ab200
