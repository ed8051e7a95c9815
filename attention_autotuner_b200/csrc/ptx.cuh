// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (TMEM alloc,
// ld/st, MMA, commit) and the UMMA shared-memory / instruction descriptors.
//
// Everything here is a one-to-one wrapper of a PTX instruction or a bit-packing helper; no policy.
// All mbarrier waits are bounded (see mbar_wait): a pipeline bug returns an error status instead of
// hanging the GPU.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ab200 {

// ----------------------------------------------------------------------------------------------
// Status word shared by every kernel of the library. 0 = ok. Non-zero values are "sticky" until
// the host clears them (attn_b200_device_status(1)).
// ----------------------------------------------------------------------------------------------
enum DeviceStatus : int {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,  // a bounded mbarrier wait expired
  kStatusSaturated = 2,    // a 16-bit intermediate hit the largest finite fp16 value: the result is not trustworthy
};

__device__ int g_device_status = 0;
__device__ int g_device_status_detail = 0;  // (barrier tag << 16) | blockIdx.x, first failure only
// Numeric flag, kept apart from g_device_status so that it never makes a wait give up: set when the RetNet forward had to
// clamp an unnormalised score to the fp16 range (see chain_common.cuh). Reported by the host as status 2.
__device__ int g_numeric_status = 0;
// Host-visible copy of the words above: mapped pinned host memory, set up once per device by the host side
// (status_mirror() in host_common.cuh). [0] = status, [1] = detail, [2] = numeric flag. The launchers read it without a
// synchronisation before every launch, so a kernel that gave up is noticed by the next call instead of silently
// poisoning everything after it. nullptr until the first launch on the device.
__device__ volatile int* g_status_mirror = nullptr;

#ifndef AB200_WAIT_LIMIT_NS
#define AB200_WAIT_LIMIT_NS 1000000000ull  // 1 s per wait
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ----------------------------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// One lane of a converged warp (elect.sync). Keeping the surrounding control flow warp-uniform and
// electing only around the instruction lets the compiler hold descriptors in uniform registers.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .b32 rx;\n\t"
      ".reg .pred px;\n\t"
      "elect.sync rx|px, %1;\n\t"
      "@px mov.s32 %0, 1;\n\t"
      "}\n"
      : "+r"(pred)
      : "r"(0xFFFFFFFFu));
  return pred != 0;
}

// Per-CTA abort word in shared memory: once any role gives up, every other bounded wait of the CTA
// returns false quickly so that all roles fall through to the common tail (TMEM free, exit).
struct CtaAbort {
  volatile int flag;
};

__device__ __noinline__ void report_timeout(CtaAbort* ab, int tag) {
  ab->flag = 1;
  if (atomicCAS(&g_device_status, kStatusOk, kStatusWaitTimeout) == kStatusOk) {
    const int detail = (tag << 16) | (blockIdx.x & 0xffff);
    g_device_status_detail = detail;
    volatile int* mirror = g_status_mirror;
    if (mirror != nullptr) {
      mirror[1] = detail;
      __threadfence_system();
      mirror[0] = kStatusWaitTimeout;
    }
  }
}

__device__ __noinline__ void report_saturation() {
  if (atomicExch(&g_numeric_status, 1) == 0) {
    volatile int* mirror = g_status_mirror;
    if (mirror != nullptr) mirror[2] = 1;
  }
}

// True when one of the two fp16 halves of `packed` is the largest finite magnitude (0x7bff), which is what
// cvt.rn.satfinite produces for every input beyond the fp16 range.
__device__ __forceinline__ bool half2_has_maxnorm(uint32_t packed) {
  const uint32_t m = packed & 0x7fff7fffu;
  return (m & 0xffffu) == 0x7bffu || (m >> 16) == 0x7bffu;
}

// Once any CTA of any launch has reported a failure the status word stays non-zero until the host clears
// it; every later wait gives up at once, so a broken pipeline costs about one wait limit in total rather
// than one per CTA.
// Bounded wait for one thread (the single-thread producer / MMA roles). Returns false on expiry or
// when another role of the CTA already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, CtaAbort* ab, int tag,
                                          uint64_t limit_ns = AB200_WAIT_LIMIT_NS) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0 = 0;
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (ab->flag || *reinterpret_cast<volatile int*>(&g_device_status) != 0) return false;
      uint64_t now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      if (now - t0 > limit_ns) {
        report_timeout(ab, tag);
        return false;
      }
    }
  }
}

// Wait used only on the abort path to let TMA copies that are still in flight land before the CTA
// exits. Ignores the abort flag; short limit; never reports.
__device__ __forceinline__ void mbar_wait_drain(uint64_t* bar, uint32_t parity, uint64_t limit_ns) {
  const uint64_t t0 = globaltimer_ns();
  while (!mbar_try_wait(bar, parity)) {
    if (globaltimer_ns() - t0 > limit_ns) return;
  }
}

// Bounded wait for a whole, converged warp. The result is warp-uniform, so the callers can keep
// issuing .sync.aligned tcgen05 instructions afterwards without divergence.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, CtaAbort* ab, int tag,
                                               uint64_t limit_ns = AB200_WAIT_LIMIT_NS) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    bool ok = mbar_try_wait(bar, parity);
    if (__all_sync(0xffffffffu, ok)) return true;
#ifdef AB200_POLL_SLEEP
    __nanosleep(AB200_POLL_SLEEP);
#endif
    if ((it & 63u) == 63u) {
      int give_up = 0;
      if ((threadIdx.x & 31) == 0) {
        if (ab->flag || *reinterpret_cast<volatile int*>(&g_device_status) != 0) {
          give_up = 1;
        } else {
          uint64_t now = globaltimer_ns();
          if (t0 == 0) t0 = now;
          if (now - t0 > limit_ns) {
            report_timeout(ab, tag);
            give_up = 1;
          }
        }
      }
      give_up = __shfl_sync(0xffffffffu, give_up, 0);
      if (give_up) return false;
    }
  }
}

// ----------------------------------------------------------------------------------------------
// Programmatic dependent launch. A kernel launched with the programmatic-stream-serialization attribute may
// start (as SMs become free) once every CTA of the kernel before it in the stream has executed
// launch_dependents or exited; grid_dependency_wait blocks until that earlier kernel has completed and its
// writes are visible. Both are no-ops for a kernel launched the ordinary way.
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ----------------------------------------------------------------------------------------------
// TMA (tiled bulk tensor copies). Loads complete on an mbarrier (complete_tx bytes); stores use
// bulk groups. Every x coordinate passed here is a multiple of 64 elements (128 bytes).
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// Untiled bulk copy global -> shared memory of this CTA; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// Asks the L2 for one box of a tensor ahead of the load that will need it (no shared-memory destination, no completion).
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(map), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* smem_src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(map),
               "r"(smem_u32(smem_src)), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read0() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA store, UMMA reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------------------------
// tcgen05: tensor memory management
// ----------------------------------------------------------------------------------------------
// Whole warp. Writes the TMEM base address (lane 0, column c) to *smem_result.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// TMEM address = (lane << 16) | column. A warp may only touch lanes [32*(warp%4), 32*(warp%4)+32).
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// 32 lanes x 32 columns of 32-bit: thread t of the warp receives lane (lane_base + t), columns
// [col, col+32) in r[0..31].
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ----------------------------------------------------------------------------------------------
// UMMA descriptors
// ----------------------------------------------------------------------------------------------
// 32-bit instruction descriptor for kind::f16 with an fp32 accumulator.
//   [4,6) D format (1 = f32)   [7,10) A format, [10,13) B format (0 = f16, 1 = bf16)
//   [15] A major, [16] B major (0 = K-major, 1 = MN-major)   [17,23) N >> 3   [24,29) M >> 4
__host__ __device__ constexpr uint32_t umma_idesc(int M, int N, bool bf16, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(N >> 3) << 17) |
         (static_cast<uint32_t>(M >> 4) << 24);
}

// 64-bit shared-memory matrix descriptor, 128-byte swizzle, sm_100 version field = 1.
//   [0,14) address >> 4   [16,30) leading byte offset >> 4   [32,46) stride byte offset >> 4
//   [46,48) version (1)   [61,64) layout (2 = SWIZZLE_128B)
// The tile must sit in a 1024-byte aligned buffer written by TMA with SWIZZLE_128B (rows of 128
// bytes, 8-row groups of 1024 bytes).
//   K-major operand  (rows = M/N index, 64 K-elements per row):  LBO unused (1), SBO = 1024.
//   MN-major operand (rows = K index, 64 MN-elements per row):   LBO = bytes between 64-element MN
//                                                                chunks, SBO = 1024 (8 K rows).
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// The same descriptor without swizzle, for small K-major operands written by threads or by a plain bulk copy: the
// tile is made of core matrices of 8 rows x 16 bytes stored contiguously (128 bytes each);
//   LBO = bytes between the two core matrices of a 16-element K slice, SBO = bytes between 8-row groups.
__device__ __forceinline__ uint64_t umma_smem_desc_noswizzle(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  return d;
}

// D[tmem] (+)= A[smem] * B[smem]. One thread issues.
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]. A is [128 lanes x K] with two 16-bit K elements per 32-bit column.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ----------------------------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two exponentials per MUFU operation: 2^x for a pair of fp16 values, results in fp16 (subnormal results are kept).
// The input pair is what cvt.rn.f16x2 makes of x, so the relative error of a result is about ln2 * ulp_fp16(x) / 2:
// 3.4e-4 for 1 <= |x| < 2, 6.8e-4 for 2 <= |x| < 4, doubling per binade of |x|.
__device__ __forceinline__ uint32_t ex2_approx_h2(uint32_t xh2) {
  uint32_t y;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(xh2));
  return y;
}
__device__ __forceinline__ uint32_t hadd2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
// Product of two packed pairs of 16-bit floats (fp16 or bf16), rounded to nearest.
template <bool BF16>
__device__ __forceinline__ uint32_t mul2_16(uint32_t a, uint32_t b) {
  uint32_t r;
  if constexpr (BF16) {
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  } else {
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  }
  return r;
}
// The two fp16 halves of a register as a packed fp32 pair (low half first).
__device__ __forceinline__ uint64_t h2_to_f2(uint32_t h2) {
  float lo, hi;
  asm("{\n\t"
      ".reg .b16 l, h;\n\t"
      "mov.b32 {l, h}, %2;\n\t"
      "cvt.f32.f16 %0, l;\n\t"
      "cvt.f32.f16 %1, h;\n\t"
      "}\n"
      : "=f"(lo), "=f"(hi)
      : "r"(h2));
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
// Three-input maximum and packed two-wide fp32 arithmetic (sm_100): halve the instruction count of the
// element-wise phases.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

__device__ __forceinline__ uint64_t fsub2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
// 2^x for a packed pair on the FMA pipes (no MUFU): floor(x) by a round-down magic-number add, a cubic
// for 2^frac on [0,1) (max relative error 8.7e-5, below the rounding step of a 16-bit result), and the
// integer part added to the exponent field. x is clamped at -126 (results below 2^-126 are not needed).
__device__ __forceinline__ void exp2_poly2(uint64_t x2, float& e0, float& e1) {
  float x0, x1;
  f2_unpack(x2, x0, x1);
  x0 = fmaxf(x0, -126.0f);
  x1 = fmaxf(x1, -126.0f);
  const uint64_t xc = f2_pack(x0, x1);
  const uint64_t magic = f2_pack(12582912.0f, 12582912.0f);  // 1.5 * 2^23
  uint64_t t;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(t) : "l"(xc), "l"(magic));
  const uint64_t fr = fsub2(xc, fsub2(t, magic));
  uint64_t pl = ffma2(fr, f2_pack(0.07705805f, 0.07705805f), f2_pack(0.22764558f, 0.22764558f));
  pl = ffma2(pl, fr, f2_pack(0.69512289f, 0.69512289f));
  pl = ffma2(pl, fr, f2_pack(1.0f, 1.0f));
  float p0, p1, t0, t1;
  f2_unpack(pl, p0, p1);
  f2_unpack(t, t0, t1);
  e0 = __uint_as_float(__float_as_uint(p0) + (__float_as_uint(t0) << 23));
  e1 = __uint_as_float(__float_as_uint(p1) + (__float_as_uint(t1) << 23));
}

// 256-bit global store (sm_100): one full 32-byte sector per lane. The address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t* r) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(ptr), "r"(r[0]), "r"(r[1]), "r"(r[2]),
               "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}

// Packs two fp32 into one 32-bit register of two 16-bit floats: low half = lo, high half = hi.
template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  uint32_t r;
  if constexpr (BF16) {
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  } else {
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  }
  return r;
}

}  // namespace ab200
