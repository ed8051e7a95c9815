// CTA-pair (cta_group::2) building-block test: the two-GEMM chain in miniature on one cluster of two CTAs.
//   Z[256,128]  = A[256,K] * B[128,K]^T      A, B K-major in shared memory; each CTA holds its 128 rows of A
//                                            and 64 rows of B
//   W           = 16-bit copy of Z           written back to tensor memory by each CTA for its own 128 rows
//   D[256,N2]   = W[256,128] * T[128,N2]     W from tensor memory, T MN-major; each CTA holds N2/2 columns
// Both Z and D are returned so that a layout mistake in either step shows up against a plain matmul.
#pragma once

#include "host_common.cuh"
#include "ptx_pair.cuh"

namespace ab200 {

constexpr int kPairSelftestSmem = 1024 + 65536 + 32768 + 32768 + 256;

template <bool BF16>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(160, 1)
selftest_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const __grid_constant__ CUtensorMap tmT, float* z_out, float* d_out, int K, int N2) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;                   // own 128 rows of A: K/64 boxes of 16 KB
  uint8_t* sB = smem + 65536;           // own 64 rows of B:  K/64 boxes of 8 KB
  uint8_t* sT = smem + 65536 + 32768;   // own N2/2 columns of T: N2/128 boxes of 16 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 65536 + 65536);
  uint64_t* ld_full = bars;      // own loads landed (transaction count)
  uint64_t* ready = bars + 1;    // leader: both CTAs' loads landed (2 arrivals)
  uint64_t* z_full = bars + 2;   // both: GEMM1 complete
  uint64_t* w_full = bars + 3;   // leader: W written by all 256 threads of the pair
  uint64_t* d_full = bars + 4;   // both: GEMM2 complete
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_slot + 1);
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const uint32_t rank = cluster_ctarank();

  if (threadIdx.x == 0) {
    mbar_init(ld_full, 1);
    mbar_init(ready, 2);
    mbar_init(z_full, 1);
    mbar_init(w_full, 256);
    mbar_init(d_full, 1);
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc2(tmem_slot, 512);
    tmem_relinquish2();
  }
  tc_fence_before();
  cluster_sync();  // barriers of both CTAs are initialised before anyone arrives remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tZ = tmem_base;
  const uint32_t tD = tmem_base + 256;

  bool ok = true;
  if (warp == 4) {
    // control warp: loads of this CTA, then (leader only) the MMAs
    if (elect_one()) {
      mbar_expect_tx(ld_full, (128 + 64) * K * 2 + 128 * (N2 / 2) * 2);
      for (int c = 0; c < K / 64; ++c) {
        tma_load_3d(sA + c * 16384, &tmA, ld_full, c * 64, rank * 128, 0);
        tma_load_3d(sB + c * 8192, &tmB, ld_full, c * 64, rank * 64, 0);
      }
      for (int c = 0; c < N2 / 128; ++c) tma_load_3d(sT + c * 16384, &tmT, ld_full, rank * (N2 / 2) + c * 64, 0, 0);
    }
    __syncwarp();
    ok = mbar_wait_warp(ld_full, 0, ab, 1);
    if (ok && elect_one()) mbar_arrive_cluster(mapa_shared(smem_u32(ready), 0));
    __syncwarp();
    if (rank == 0 && ok) {
      ok = mbar_wait_warp(ready, 0, ab, 2);
      if (ok) {
        tc_fence_after();
        if (elect_one()) {
          const uint32_t idesc = umma_idesc(256, 128, BF16, false, false);
          for (int ks = 0; ks < K / 16; ++ks) {
            const uint32_t a = smem_u32(sA) + (ks >> 2) * 16384 + (ks & 3) * 32;
            const uint32_t b = smem_u32(sB) + (ks >> 2) * 8192 + (ks & 3) * 32;
            umma_ss2(tZ, umma_smem_desc(a, 16, 1024), umma_smem_desc(b, 16, 1024), idesc, ks > 0 ? 1u : 0u);
          }
          tc_commit2_both(z_full);
        }
        __syncwarp();
        ok = mbar_wait_warp(w_full, 0, ab, 4);
      }
      if (ok) {
        tc_fence_after();
        if (elect_one()) {
          const uint32_t idesc = umma_idesc(256, N2, BF16, false, true);
          for (int ks = 0; ks < 8; ++ks)
            umma_ts2(tD, tZ + ks * 8, umma_smem_desc(smem_u32(sT) + ks * 2048, 16384, 1024), idesc, ks > 0 ? 1u : 0u);
          tc_commit2_both(d_full);
        }
        __syncwarp();
      }
    }
  } else {
    // 128 threads: thread t owns TMEM lane t = row rank*128 + t of Z, W and D
    const int row = rank * 128 + threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32);
    ok = mbar_wait_warp(z_full, 0, ab, 3);
    if (ok) {
      tc_fence_after();
      const uint32_t tz = tmem_addr(tZ, lane_base, 0);
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t r[32];
        tmem_ld32(tz + qd * 32, r);
        tc_wait_ld();
        uint32_t pk[16];
        for (int i = 0; i < 32; i += 2) {
          z_out[row * 128 + qd * 32 + i] = __uint_as_float(r[i]);
          z_out[row * 128 + qd * 32 + i + 1] = __uint_as_float(r[i + 1]);
          pk[i >> 1] = pack2<BF16>(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        }
        tmem_st16(tz + qd * 16, pk);  // overlays columns that were read in this or an earlier chunk
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive_cluster(mapa_shared(smem_u32(w_full), 0));
      ok = mbar_wait_warp(d_full, 0, ab, 5);
    }
    if (ok) {
      tc_fence_after();
      const uint32_t td = tmem_addr(tD, lane_base, 0);
      for (int c0 = 0; c0 < N2; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(td + c0, r);
        tc_wait_ld();
        for (int i = 0; i < 32; ++i) d_out[row * N2 + c0 + i] = __uint_as_float(r[i]);
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  cluster_sync();  // no CTA leaves while the other may still arrive on its barriers or read its shared memory
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, 512);
  }
}

// a: [256,K], b: [128,K], t: [128,N2] 16-bit row-major; z: [256,128], d: [256,N2] fp32.
// K in {64,128,192,256}, N2 in {128,256}.
inline int selftest_pair(const void* a, const void* b, const void* t, float* z, float* d, int K, int N2, int bf16,
                         cudaStream_t stream) {
  if (!a || !b || !t || !z || !d) return fail(kErrInvalidArgument, "selftest_pair: null pointer");
  if (K % 64 != 0 || K < 64 || K > 256 || (N2 != 128 && N2 != 256))
    return fail(kErrInvalidArgument, "selftest_pair: unsupported K=%d N2=%d", K, N2);
  CUtensorMap ta, tb, tt;
  int rc;
  if ((rc = bind_device_of(a, "selftest_pair"))) return rc;
  if ((rc = make_tmap_3d(&ta, a, bf16 != 0, K, 256, 1, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tb, b, bf16 != 0, K, 128, 1, 64, 64))) return rc;
  if ((rc = make_tmap_3d(&tt, t, bf16 != 0, N2, 128, 1, 64, 128))) return rc;
  auto launch = [&](auto kernel) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSelftestSmem);
    kernel<<<2, 160, kPairSelftestSmem, stream>>>(ta, tb, tt, z, d, K, N2);
  };
  if (bf16) launch(selftest_pair_kernel<true>); else launch(selftest_pair_kernel<false>);
  return check_launch("selftest_pair");
}

}  // namespace ab200
