// Single-CTA GEMM kernels that exercise, in isolation, each tcgen05/TMA building block the
// attention kernels are made of. They exist so that a descriptor or layout mistake shows up as a
// failing 128xN GEMM against a plain matmul rather than as a wrong attention output.
//   ss: D[128,N] = A[128,K] * B[N,K]^T   A, B K-major in shared memory (the Q K^T step)
//   ts: D[128,N] = P[128,128] * V[128,N] P in tensor memory, V MN-major in shared memory (the P V step)
#pragma once

#include "host_common.cuh"
#include "ptx.cuh"

namespace ab200 {

constexpr int kSelftestSmem = 2 * 65536 + 1024 + 64;

__global__ void __launch_bounds__(128, 1)
selftest_gemm_ss_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, float* d,
                        int N, int K, int bf16) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + 65536;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * 65536);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  bool ok = true;
  if (threadIdx.x == 0) {
    mbar_expect_tx(&bars[0], (128 + N) * K * 2);
    for (int c = 0; c < K / 64; ++c) {
      tma_load_3d(sA + c * (128 * 128), &tmA, &bars[0], c * 64, 0, 0);
      tma_load_3d(sB + c * (N * 128), &tmB, &bars[0], c * 64, 0, 0);
    }
    ok = mbar_wait(&bars[0], 0, ab, 1);
    if (ok) {
      tc_fence_after();
      const uint32_t idesc = umma_idesc(128, N, bf16 != 0, false, false);
      for (int ks = 0; ks < K / 16; ++ks) {
        const uint32_t a = smem_u32(sA) + (ks >> 2) * (128 * 128) + (ks & 3) * 32;
        const uint32_t b = smem_u32(sB) + (ks >> 2) * (N * 128) + (ks & 3) * 32;
        umma_ss(tmem_base, umma_smem_desc(a, 16, 1024), umma_smem_desc(b, 16, 1024), idesc, ks > 0 ? 1u : 0u);
      }
      tc_commit(&bars[1]);
    }
  }
  __syncwarp();
  ok = mbar_wait_warp(&bars[1], 0, ab, 2);
  if (ok) {
    tc_fence_after();
    const uint32_t t = tmem_addr(tmem_base, warp * 32, 0);
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(t + c0, r);
      tc_wait_ld();
      for (int i = 0; i < 32; ++i) d[threadIdx.x * N + c0 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

__global__ void __launch_bounds__(128, 1)
selftest_gemm_ts_kernel(const uint32_t* p_packed /*[128][64] two 16-bit per word*/,
                        const __grid_constant__ CUtensorMap tmV, float* d, int N, int bf16) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sV = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * 65536);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5;

  if (threadIdx.x == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tP = tmem_base;        // columns [0, 64)
  const uint32_t tD = tmem_base + 256;  // columns [256, 256+N)

  // every thread writes its row of P into tensor memory
  {
    uint32_t r[32];
    const uint32_t t = tmem_addr(tP, warp * 32, 0);
    for (int h = 0; h < 2; ++h) {
      for (int i = 0; i < 32; ++i) r[i] = p_packed[threadIdx.x * 64 + h * 32 + i];
      tmem_st32(t + h * 32, r);
    }
    tc_wait_st();
  }
  tc_fence_before();
  __syncthreads();

  bool ok = true;
  if (threadIdx.x == 0) {
    tc_fence_after();
    mbar_expect_tx(&bars[0], 128 * N * 2);
    for (int c = 0; c < N / 64; ++c) tma_load_3d(sV + c * (128 * 128), &tmV, &bars[0], c * 64, 0, 0);
    ok = mbar_wait(&bars[0], 0, ab, 1);
    if (ok) {
      tc_fence_after();
      const uint32_t idesc = umma_idesc(128, N, bf16 != 0, false, true);
      for (int ks = 0; ks < 8; ++ks)
        umma_ts(tD, tP + ks * 8, umma_smem_desc(smem_u32(sV) + ks * 2048, 128 * 128, 1024), idesc, ks > 0 ? 1u : 0u);
      tc_commit(&bars[1]);
    }
  }
  __syncwarp();
  ok = mbar_wait_warp(&bars[1], 0, ab, 2);
  if (ok) {
    tc_fence_after();
    const uint32_t t = tmem_addr(tD, warp * 32, 0);
    for (int c0 = 0; c0 < N; c0 += 32) {
      uint32_t r[32];
      tmem_ld32(t + c0, r);
      tc_wait_ld();
      for (int i = 0; i < 32; ++i) d[threadIdx.x * N + c0 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// a: [128,K], b: [N,K], d: [128,N] fp32. K in {64,128,192,256}, N multiple of 32 in [32,256].
inline int selftest_gemm_ss(const void* a, const void* b, float* d, int N, int K, int bf16, cudaStream_t stream) {
  if (!a || !b || !d) return fail(kErrInvalidArgument, "selftest_gemm_ss: null pointer");
  if (K % 64 != 0 || K < 64 || K > 256 || N % 32 != 0 || N < 32 || N > 256 || N * K > 32768)
    return fail(kErrInvalidArgument, "selftest_gemm_ss: unsupported N=%d K=%d", N, K);
  CUtensorMap ta, tb;
  int rc;
  if ((rc = bind_device_of(a, "selftest_gemm_ss"))) return rc;
  if ((rc = make_tmap_3d(&ta, a, bf16 != 0, K, 128, 1, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tb, b, bf16 != 0, K, N, 1, 64, N))) return rc;
  cudaFuncSetAttribute(selftest_gemm_ss_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelftestSmem);
  selftest_gemm_ss_kernel<<<1, 128, kSelftestSmem, stream>>>(ta, tb, d, N, K, bf16);
  return check_launch("selftest_gemm_ss");
}

// p: [128,128] 16-bit, v: [128,N] 16-bit row-major, d: [128,N] fp32. N multiple of 64 in [64,256].
inline int selftest_gemm_ts(const void* p, const void* v, float* d, int N, int bf16, cudaStream_t stream) {
  if (!p || !v || !d) return fail(kErrInvalidArgument, "selftest_gemm_ts: null pointer");
  if (N % 64 != 0 || N < 64 || N > 256) return fail(kErrInvalidArgument, "selftest_gemm_ts: unsupported N=%d", N);
  CUtensorMap tv;
  int rc;
  if ((rc = bind_device_of(v, "selftest_gemm_ts"))) return rc;
  if ((rc = make_tmap_3d(&tv, v, bf16 != 0, N, 128, 1, 64, 128))) return rc;
  cudaFuncSetAttribute(selftest_gemm_ts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelftestSmem);
  selftest_gemm_ts_kernel<<<1, 128, kSelftestSmem, stream>>>(reinterpret_cast<const uint32_t*>(p), tv, d, N, bf16);
  return check_launch("selftest_gemm_ts");
}

// The bounded wait in miniature: one warp waits on an mbarrier that nobody ever arrives at, with a wait limit of
// limit_ns instead of the kernels' one second. The wait runs out, report_timeout() sets the status words and the kernel
// returns normally: no TMA, no tensor memory, no cluster, nothing in flight. whole_warp selects mbar_wait_warp
// (the converged-warp form the MMA and softmax roles use) or mbar_wait (the single-thread form of the producers).
constexpr int kTagSelftestWait = 99;
__global__ void __launch_bounds__(32, 1) selftest_wait_kernel(unsigned long long limit_ns, int whole_warp) {
  __shared__ uint64_t bar;
  __shared__ CtaAbort ab;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    ab.flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  if (whole_warp) {
    (void)mbar_wait_warp(&bar, 0, &ab, kTagSelftestWait, limit_ns);
  } else if (threadIdx.x == 0) {
    (void)mbar_wait(&bar, 0, &ab, kTagSelftestWait, limit_ns);
  }
}

inline int selftest_wait(int limit_us, int whole_warp, cudaStream_t stream) {
  if (limit_us <= 0 || limit_us > 100000) return fail(kErrInvalidArgument, "selftest_wait: limit_us must be in [1, 100000]");
  if (int prior = check_prior_status("selftest_wait")) return prior;
  selftest_wait_kernel<<<1, 32, 0, stream>>>(static_cast<unsigned long long>(limit_us) * 1000ull, whole_warp ? 1 : 0);
  return check_launch("selftest_wait");
}

}  // namespace ab200
