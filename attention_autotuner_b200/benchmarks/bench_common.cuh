// Shared pieces of the standalone C++ micro-benchmarks (attention.cu, retnet.cu): problem shapes, named tile
// configurations, seeded N(0,1) inputs generated on the device, and the timing loop.
//
// Same roles as the reference's benchmarks/configs.h (ProblemShape and the ImplementShape* tile records,
// :3-128) and benchmarks/do_bench.cuh:8-63 (one untimed call, a five-call estimate, 50 ms of warm-up, then about
// 100 ms of launches each with its own event pair and a 256 MB buffer rewritten before it). The tile records are
// the sm_100a kernels' own template configurations instead of the reference's Br/Bc/warp-grid tuples, and the
// timing result carries the median next to the reference's mean.
#pragma once

#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <functional>
#include <string>
#include <vector>

struct ProblemShape {
  int B, H, Seq_q, Seq_k;
  ProblemShape(int b = 4, int h = 8, int sq = 2048, int sk = 2048) : B(b), H(h), Seq_q(sq), Seq_k(sk) {}
};

struct BenchResult {
  float mean_ms = -1.f, median_ms = -1.f, min_ms = -1.f;
  int repeats = 0;
};

#define BENCH_CUDA(call)                                                                         \
  do {                                                                                           \
    cudaError_t e_ = (call);                                                                     \
    if (e_ != cudaSuccess) {                                                                     \
      fprintf(stderr, "%s:%d: %s: %s\n", __FILE__, __LINE__, #call, cudaGetErrorString(e_));     \
      exit(2);                                                                                   \
    }                                                                                            \
  } while (0)

// Times launch() on the default stream. launch() returns 0 on success.
inline BenchResult do_bench(const std::function<int()>& launch, float ms_warmup = 50.f, float ms_measure = 100.f) {
  BenchResult res;
  const size_t flush_bytes = 256u * 1000u * 1000u;  // larger than the 126 MB L2
  void* flush = nullptr;
  BENCH_CUDA(cudaMalloc(&flush, flush_bytes));
  cudaEvent_t a, b;
  BENCH_CUDA(cudaEventCreate(&a));
  BENCH_CUDA(cudaEventCreate(&b));
  if (launch() != 0) return res;
  BENCH_CUDA(cudaEventRecord(a, 0));
  for (int i = 0; i < 5; ++i)
    if (launch() != 0) return res;
  BENCH_CUDA(cudaEventRecord(b, 0));
  BENCH_CUDA(cudaEventSynchronize(b));
  float est = 0.f;
  BENCH_CUDA(cudaEventElapsedTime(&est, a, b));
  est = std::max(est / 5.f, 1e-3f);
  const int n_warm = std::max(1, static_cast<int>(ceilf(ms_warmup / est)));
  const int n_rep = std::min(2000, std::max(3, static_cast<int>(ceilf(ms_measure / est))));
  for (int i = 0; i < n_warm; ++i)
    if (launch() != 0) return res;
  std::vector<cudaEvent_t> starts(n_rep), stops(n_rep);
  for (int i = 0; i < n_rep; ++i) {
    BENCH_CUDA(cudaEventCreate(&starts[i]));
    BENCH_CUDA(cudaEventCreate(&stops[i]));
  }
  for (int i = 0; i < n_rep; ++i) {
    BENCH_CUDA(cudaMemsetAsync(flush, i & 0xff, flush_bytes, 0));
    BENCH_CUDA(cudaEventRecord(starts[i], 0));
    if (launch() != 0) return res;
    BENCH_CUDA(cudaEventRecord(stops[i], 0));
  }
  BENCH_CUDA(cudaDeviceSynchronize());
  std::vector<float> ms(n_rep);
  double sum = 0.0;
  for (int i = 0; i < n_rep; ++i) {
    BENCH_CUDA(cudaEventElapsedTime(&ms[i], starts[i], stops[i]));
    sum += ms[i];
    cudaEventDestroy(starts[i]);
    cudaEventDestroy(stops[i]);
  }
  std::sort(ms.begin(), ms.end());
  res.mean_ms = static_cast<float>(sum / n_rep);
  res.median_ms = (n_rep & 1) ? ms[n_rep / 2] : 0.5f * (ms[n_rep / 2 - 1] + ms[n_rep / 2]);
  res.min_ms = ms[0];
  res.repeats = n_rep;
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  cudaFree(flush);
  return res;
}

// Seeded N(0, sigma) 16-bit values: element i is a pure function of (seed, i) (hash -> two uniforms -> Box-Muller),
// so a tensor is reproducible whatever the grid that fills it. The reference draws from thrust::default_random_engine
// with discard(n) per element (benchmarks/attention.cu:19-31).
__device__ __forceinline__ uint32_t bench_hash(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
template <bool BF16>
__global__ void bench_fill_normal(uint16_t* out, size_t n, uint32_t seed, float sigma) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const uint32_t lo = static_cast<uint32_t>(i), hi = static_cast<uint32_t>(i >> 32);
    const uint32_t h1 = bench_hash(lo * 2u + 1u + seed * 0x9e3779b9U + hi * 0x85ebca6bU);
    const uint32_t h2 = bench_hash(h1 ^ (lo * 2u + 0x68bc21ebU));
    const float u1 = (static_cast<float>(h1 >> 8) + 1.0f) * (1.0f / 16777217.0f);  // (0, 1)
    const float u2 = static_cast<float>(h2 >> 8) * (1.0f / 16777216.0f);
    const float v = sigma * sqrtf(-2.0f * __logf(u1)) * __cosf(6.2831853f * u2);
    if (BF16) out[i] = __bfloat16_as_ushort(__float2bfloat16(v));
    else out[i] = __half_as_ushort(__float2half(v));
  }
}
inline void fill_normal(void* ptr, size_t n, uint32_t seed, bool bf16, float sigma = 1.0f) {
  const int blocks = 148 * 8;
  if (bf16) bench_fill_normal<true><<<blocks, 256>>>(static_cast<uint16_t*>(ptr), n, seed, sigma);
  else bench_fill_normal<false><<<blocks, 256>>>(static_cast<uint16_t*>(ptr), n, seed, sigma);
  BENCH_CUDA(cudaGetLastError());
}

// lower-triangular decay mask M[h][i][j] = gamma_h^(i-j), gamma_h = 1 - 2^(-5-h), as a 16-bit tensor
template <bool BF16>
__global__ void bench_fill_decay_mask(uint16_t* out, int H, int Lq, int Lkv) {
  const size_t n = static_cast<size_t>(H) * Lq * Lkv;
  for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < n; idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const int j = static_cast<int>(idx % Lkv);
    const int i = static_cast<int>((idx / Lkv) % Lq);
    const int h = static_cast<int>(idx / (static_cast<size_t>(Lkv) * Lq));
    const float gamma = 1.0f - exp2f(-5.0f - h);
    const float v = (i >= j) ? exp2f((i - j) * log2f(gamma)) : 0.0f;
    if (BF16) out[idx] = __bfloat16_as_ushort(__float2bfloat16(v));
    else out[idx] = __half_as_ushort(__float2half(v));
  }
}

inline double attention_pairs(int Lq, int Lkv, bool causal) {
  if (!causal) return static_cast<double>(Lq) * Lkv;
  double p = 0.0;
  for (int i = 0; i < Lq; ++i) p += std::max(0, std::min(Lkv, i + (Lkv - Lq) + 1));
  return p;
}

// "--name value" / "--flag" command lines
struct Args {
  int argc;
  char** argv;
  bool flag(const char* name) const {
    for (int i = 1; i < argc; ++i)
      if (!strcmp(argv[i], name)) return true;
    return false;
  }
  int num(const char* name, int dflt) const {
    for (int i = 1; i + 1 < argc; ++i)
      if (!strcmp(argv[i], name)) return atoi(argv[i + 1]);
    return dflt;
  }
  std::string str(const char* name, const char* dflt) const {
    for (int i = 1; i + 1 < argc; ++i)
      if (!strcmp(argv[i], name)) return argv[i + 1];
    return dflt;
  }
};

inline void print_result(const char* what, const char* config, const ProblemShape& s, int dqk, int dv, const BenchResult& r, double flops) {
  if (r.mean_ms <= 0.f) {
    printf("%s [%s] B=%d H=%d Seq_q=%d Seq_k=%d Kd=%d D=%d: FAILED\n", what, config, s.B, s.H, s.Seq_q, s.Seq_k, dqk, dv);
    return;
  }
  // first the reference's line ("Time: <mean>ms", benchmarks/attention.cu:288), then the detail
  printf("Time: %gms\n", r.mean_ms);
  printf("%s [%s] B=%d H=%d Seq_q=%d Seq_k=%d Kd=%d D=%d: mean %.4f ms, median %.4f ms, min %.4f ms over %d launches, %.1f TFLOP/s (median)\n",
         what, config, s.B, s.H, s.Seq_q, s.Seq_k, dqk, dv, r.mean_ms, r.median_ms, r.min_ms, r.repeats,
         flops / (r.median_ms * 1e-3) / 1e12);
}
