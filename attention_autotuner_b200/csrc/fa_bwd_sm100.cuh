// Flash-attention backward for sm_100a, one kernel per gradient (the dQ flavour is the last launch of every backward;
// dV and dK run only where fa_bwd_kv_sm100.cuh does not): three kernels that each own their output tile (no atomics, no fp32
// accumulation buffer in global memory, bit-reproducible), built on the two-GEMM chain skeleton of chain_sm100.cuh
// with a second "GEMM1" where the element-wise step needs both S and dP:
//
//     Z1[128,128] = R1[128,D] * C1_t[128,D]^T                       (S or S^T; K-major operands in shared memory)
//     Z2[128,128] = R2[128,D] * C2_t[128,D]^T                       (dP or dP^T; dK and dQ kernels only)
//     W           = f(Z1, Z2)                                       (registers; 16-bit, written over Z1 in TMEM)
//     ACC[128,D] += W[128,128] * T_t[128,D]                         (W from tensor memory, T_t MN-major in smem)
//
//   kernel  rows     R1  R2   C1_t  C2_t  T_t   W
//   dV      keys     K   -    Q     -     dO    P^T,  P = exp(scale*S - lse[query])
//   dK      keys     K   V    Q     dO    Q     P^T .* (dP^T - delta[query]) * scale
//   dQ      queries  Q   dO   K     V     K     P   .* (dP   - delta[query]) * scale
//
// with delta[i] = sum_d dO[i,d] * O[i,d], computed inside the kernels from the rows of dO and O (the dQ kernel: the
// thread's own row, once per tile; the dK kernel: 128 rows per block, by the helper warpgroup).
// The reference has no attention backward (python/ops/attention_interface.py:38-39 is `pass`); the formulas are the
// derivative of its forward (python/utils/ref_op.py:2-6) with the softmax recomputed from the forward's log-sum-exp.
//
// Roles: warps 0-3 and 8-11 are two element-wise warpgroups (two threads per row of the block: columns 0-63 and
// 64-127), warp 4 issues both GEMM1s, warp 5 GEMM2, warp 6 lane 0 is the TMA producer, warps 12-15 are the helper
// warpgroup: it writes the accumulator out when a tile is finished and, in the kernels whose columns are queries,
// prepares the per-column terms (-lse * log2 e and -delta * scale) of the coming blocks in a small ring of tables in
// shared memory, so that the element-wise threads never wait for global memory. Every streamed tile is one ring item
// (two boxes of 128 rows x 64 columns for D = 128), so the MMA warps wait on the ring barriers themselves. Tensor
// memory: Z1 double buffered at columns [0,256), Z2 single at [256,384) (dV kernel: a third Z1 buffer), ACC at
// [384,384+D). W (16-bit) overlays Z1:
// columns 0-63 of the block at [0,32), columns 64-127 at [64,96) of the buffer, each half written by the warpgroup
// that read it.
#pragma once

#include "ptx.cuh"

namespace ab200 {

enum FaBwdWhich : int { kFaBwdDV = 0, kFaBwdDK = 1, kFaBwdDQ = 2 };

struct FaBwdParams {
  void* out;           // [BH, rows, D] 16-bit
  const float* lse;    // [BH, Lq] natural-log log-sum-exp of scale * S, from the forward
  const void* o;       // [BH, Lq, D] forward output   (delta; dK and dQ kernels)
  const void* dout;    // [BH, Lq, D] its gradient     (delta; dK and dQ kernels)
  int Lq, Lkv;
  float scale;
  int causal;          // 1: Lq == Lkv and key j > query i masked; blocks above the diagonal are skipped
  int nrb;             // 128-row blocks on the row side
  int total_items;     // nrb * BH
};

struct FaBwdItem {
  int bh, row0, t_start, n_iter;
};

enum FaBwdTag : int {
  kFbR = 31, kFbSlotFull = 32, kFbSlotEmpty = 33, kFbZFull = 34, kFbWFull = 35, kFbAccDone = 36, kFbAccFree = 37,
  kFbRFree = 38, kFbZFree = 39, kFbZ2Full = 40, kFbZ2Free = 41, kFbTabFull = 42, kFbTabFree = 43
};

// Optional event trace (compile with -DAB200_TRACE): clock64 of CTA 0 at the hand-over points of the first blocks.
#ifdef AB200_TRACE
constexpr int kFaBwdTraceIters = 48;
__device__ long long g_fa_bwd_trace[3][kFaBwdTraceIters][8];
#define AB200_FBTR(who, j, ev)                                                                     \
  do {                                                                                             \
    if (blockIdx.x == 0 && (j) < kFaBwdTraceIters) g_fa_bwd_trace[who][j][ev] = clock64();         \
  } while (0)
#else
#define AB200_FBTR(who, j, ev) do {} while (0)
#endif

template <int D_, int WHICH_, bool BF16_>
struct FaBwdConfig {
  static constexpr int D = D_;  // head dimension of q, k, v (64 or 128)
  static constexpr int WHICH = WHICH_;
  static constexpr bool BF16 = BF16_;
  static constexpr bool DUAL = WHICH != kFaBwdDV;
  static constexpr bool ROWK = WHICH != kFaBwdDQ;  // rows of the tile are keys
  static constexpr int DB = D / 64;                // boxes per tile
  static constexpr int BOX_BYTES = 128 * 128;
  static constexpr int ITEM_BYTES = 2 * BOX_BYTES;
  static constexpr int R_BYTES = 128 * D * 2;
  static constexpr int NR = DUAL ? 2 : 1;          // resident tiles
  static constexpr int NC = DUAL ? 2 : 1;          // C tiles per block
  static constexpr int NTAB = 4;                   // ring of per-block column tables (2 x 128 floats each)
  // dK kernel: -delta * scale of the first DCACHE_BLOCKS query blocks of the slice the helper worked on last; the two
  // work items of a pair belong to the same slice, so the second one finds its values here
  static constexpr int DCACHE_BLOCKS = (WHICH == kFaBwdDK) ? 32 : 0;
  static constexpr int AUX_BYTES = NTAB * 1024 + 1024 + DCACHE_BLOCKS * 512;  // tables, barriers and flags, delta cache
  static constexpr int NSLOT_FIT = (232448 - 1024 - AUX_BYTES - NR * R_BYTES) / ITEM_BYTES;
  static constexpr int NSLOT = NSLOT_FIT > 5 ? 5 : NSLOT_FIT;
  static constexpr int SMEM_BYTES = 1024 + NR * R_BYTES + NSLOT * ITEM_BYTES + AUX_BYTES;
  static constexpr int NTHREADS = 512;
  static constexpr int TMEM_COLS = 512;
  static_assert(D == 64 || D == 128, "head dimension");
  static_assert(NSLOT >= 4, "ring too small");
};

// delta[row] = sum_d dO[row,d] * O[row,d] (fp32 accumulation of 16-bit inputs) for the 32 consecutive query rows
// row0 ... row0 + 31 of slice bh, computed by one converged warp with coalesced 16-byte loads (D / 8 lanes per row,
// butterfly reduction); lane l returns the value of row row0 + l, 0 for rows past Lq.
template <int D, bool BF16>
__device__ __forceinline__ float fa_bwd_delta_warp(const void* o, const void* dout, int bh, int row0, int Lq, int lane) {
  constexpr int LPR = D / 8;     // lanes per row
  constexpr int RPI = 32 / LPR;  // rows per iteration
  const uint16_t* po = reinterpret_cast<const uint16_t*>(o);
  const uint16_t* pd = reinterpret_cast<const uint16_t*>(dout);
  float mine = 0.f;
  // Eight iterations' loads (16 x 16 bytes per lane) are issued before the first use: the loop is bound by the
  // latency of global memory, not by its bandwidth.
  constexpr int NIT = 32 / RPI, BATCH = NIT < 8 ? NIT : 8;
#pragma unroll 1
  for (int it0 = 0; it0 < NIT; it0 += BATCH) {
    uint4 a[BATCH], b[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const int row = row0 + (it0 + i) * RPI + lane / LPR;
      a[i] = make_uint4(0, 0, 0, 0);
      b[i] = make_uint4(0, 0, 0, 0);
      if (row < Lq) {
        const size_t off = (static_cast<size_t>(bh) * Lq + row) * D + (lane % LPR) * 8;
        a[i] = __ldg(reinterpret_cast<const uint4*>(po + off));
        b[i] = __ldg(reinterpret_cast<const uint4*>(pd + off));
      }
    }
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
      const uint32_t aw[4] = {a[i].x, a[i].y, a[i].z, a[i].w}, bw[4] = {b[i].x, b[i].y, b[i].z, b[i].w};
      float s = 0.f;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float a0, a1, b0, b1;
        if (BF16) {
          a0 = __uint_as_float(aw[e] << 16);
          a1 = __uint_as_float(aw[e] & 0xffff0000u);
          b0 = __uint_as_float(bw[e] << 16);
          b1 = __uint_as_float(bw[e] & 0xffff0000u);
        } else {
          const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[e]));
          const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[e]));
          a0 = fa.x; a1 = fa.y; b0 = fb.x; b1 = fb.y;
        }
        s = fmaf(a0, b0, s);
        s = fmaf(a1, b1, s);
      }
#pragma unroll
      for (int m = LPR / 2; m >= 1; m >>= 1) s += __shfl_xor_sync(0xffffffffu, s, m);
      // row row0 + it * RPI + j is complete in lanes [j * LPR, (j + 1) * LPR); lane l keeps row l
      const float v = __shfl_sync(0xffffffffu, s, (lane % RPI) * LPR);
      if (lane / RPI == it0 + i) mine = v;
    }
  }
  return mine;
}

template <bool BF16>
__device__ __forceinline__ uint64_t fa_bwd_unpack2(uint32_t packed) {
  if constexpr (BF16) {
    return f2_pack(__uint_as_float(packed << 16), __uint_as_float(packed & 0xffff0000u));
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&packed));
    return f2_pack(f.x, f.y);
  }
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
fa_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmR1, const __grid_constant__ CUtensorMap tmR2,
                    const __grid_constant__ CUtensorMap tmC1, const __grid_constant__ CUtensorMap tmC2,
                    const __grid_constant__ CUtensorMap tmT, const FaBwdParams p) {
  constexpr int D = Cfg::D, DB = Cfg::DB, NSLOT = Cfg::NSLOT, NC = Cfg::NC, ITEM = Cfg::ITEM_BYTES, BOX = Cfg::BOX_BYTES;
  constexpr bool DUAL = Cfg::DUAL, ROWK = Cfg::ROWK, BF16 = Cfg::BF16;
  // FUSED: the element-wise step computes P and dS in one pass over the two accumulators (the dK kernel: keeping P
  // packed in registers next to the per-column terms made its first pass 2900 cycles per block against 1650 in dQ)
#ifndef AB200_FA_BWD_FUSED_DK
#define AB200_FA_BWD_FUSED_DK 1
#endif
#ifndef AB200_FA_BWD_FUSED_DQ
#define AB200_FA_BWD_FUSED_DQ 0
#endif
#ifndef AB200_FA_BWD_POLY
#define AB200_FA_BWD_POLY 0
#endif
#ifndef AB200_FA_BWD_POLY_EVERY
#define AB200_FA_BWD_POLY_EVERY 2
#endif
  constexpr bool FUSED = DUAL && (ROWK ? (AB200_FA_BWD_FUSED_DK != 0) : (AB200_FA_BWD_FUSED_DQ != 0));
  // LEAN (the dQ kernel): dS is formed as a packed 16-bit product P .* (dP - delta) and the factor `scale` is applied
  // once per output element in the epilogue instead of once per score.
  constexpr bool LEAN = !ROWK && !FUSED;
  constexpr int NZ = DUAL ? 2 : 3;   // Z1 buffers: the dV kernel has no Z2 and uses its columns for a third one
  constexpr int PER_BLOCK = NC + 1;  // ring items per 128-wide block: C1 (, C2), T

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sR1 = smem;
  uint8_t* sR2 = smem + Cfg::R_BYTES;  // only with DUAL
  uint8_t* sRing = smem + Cfg::NR * Cfg::R_BYTES;
  // [NTAB][256]: per block of 128 queries, -delta * scale at [0,128) and -lse * log2(e) at [128,256)
  float* ctab = reinterpret_cast<float*>(sRing + NSLOT * ITEM);
  uint64_t* bars = reinterpret_cast<uint64_t*>(ctab + Cfg::NTAB * 256);
  uint64_t* r_full = bars;                    // [1]
  uint64_t* slot_full = bars + 1;             // [NSLOT]
  uint64_t* slot_empty = slot_full + NSLOT;   // [NSLOT]
  uint64_t* z_full = slot_empty + NSLOT;      // [NZ] GEMM1 into Z1 buffer complete
  uint64_t* w_full = z_full + 3;              // [NZ] W written over the Z1 buffer (element-wise -> GEMM2)
  uint64_t* z_free = w_full + 3;              // [NZ] GEMM2 of a block complete: its Z1/W buffer may be rewritten
  uint64_t* z2_full = z_free + 3;             // [1] second GEMM1 complete
  uint64_t* z2_free = z2_full + 1;            // [1] Z2 read into registers (element-wise -> GEMM1 warp)
  uint64_t* acc_done = z2_free + 1;           // [1]
  uint64_t* acc_free = acc_done + 1;          // [1]
  uint64_t* r_free = acc_free + 1;            // [1]
  uint64_t* tab_full = r_free + 1;            // [NTAB] column table written            (helper -> element-wise)
  uint64_t* tab_free = tab_full + Cfg::NTAB;  // [NTAB] column table read into registers (element-wise -> helper)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tab_free + Cfg::NTAB);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 2);
  float* dcache = reinterpret_cast<float*>(sRing + NSLOT * ITEM + Cfg::NTAB * 1024 + 1024);  // [DCACHE_BLOCKS][128]

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  const int rows_len = ROWK ? p.Lkv : p.Lq;
  const int cols_len = ROWK ? p.Lq : p.Lkv;
  const int ncb = (cols_len + 127) / 128;
  auto decode = [&](int w) -> FaBwdItem {
    FaBwdItem it;
    const int k = w % p.nrb;
    it.bh = w / p.nrb;
    const int rb = (p.causal && !ROWK) ? (p.nrb - 1 - k) : k;  // heaviest row blocks first
    it.row0 = rb * 128;
    it.t_start = 0;
    it.n_iter = ncb;
    if (p.causal) {
      if (ROWK) {
        it.t_start = rb;  // query blocks before this key block see none of its keys
        it.n_iter = ncb - rb;
      } else {
        it.n_iter = (rb + 1 < ncb) ? rb + 1 : ncb;
      }
      if (it.n_iter < 0) it.n_iter = 0;
    }
    return it;
  };
  // Work list: pairs (k-th heaviest, k-th lightest row block of a slice), as in chain_sm100.cuh, handed out round-robin
  // in runs of G consecutive pairs per CTA. G = 1 keeps all CTAs on neighbouring slices (operands shared in L2); the
  // dK kernel takes G = 2, i.e. four tiles of one slice in a row, so that its helper finds three of four delta
  // tables in its cache (computing one takes about 5300 cycles, against 3200 for the rest of a block).
  constexpr int G = (Cfg::WHICH == kFaBwdDK) ? 2 : 1;
  const int npair = (p.nrb + 1) / 2;
  const int n_super = (p.total_items / p.nrb) * npair;
  const int per_window = static_cast<int>(gridDim.x) * G;
  const int n_steps = 2 * G * ((n_super + per_window - 1) / per_window);
  auto decode_step = [&](int u, FaBwdItem& it) -> bool {
    const int s = u >> 1;
    const int sidx = ((s / G) * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x)) * G + (s % G);
    if (sidx >= n_super) return false;
    const int j = sidx % npair;
    const int k = (u & 1) ? p.nrb - 1 - j : j;
    if ((u & 1) && k == j) return false;
    it = decode((sidx / npair) * p.nrb + k);
    return true;
  };

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    for (int i = 0; i < NSLOT; ++i) {
      mbar_init(&slot_full[i], 1);
      mbar_init(&slot_empty[i], 1);
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(&z_full[i], 1);
      mbar_init(&w_full[i], 256);
      mbar_init(&z_free[i], 1);
    }
    for (int i = 0; i < Cfg::NTAB; ++i) {
      mbar_init(&tab_full[i], 128);
      mbar_init(&tab_free[i], 256);
    }
    mbar_init(z2_full, 1);
    mbar_init(z2_free, 256);
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 128);
    mbar_init(r_free, 1);
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 6 && lane == 0) {
    tma_prefetch_desc(&tmR1);
    tma_prefetch_desc(&tmC1);
    tma_prefetch_desc(&tmT);
    if (DUAL) {
      tma_prefetch_desc(&tmR2);
      tma_prefetch_desc(&tmC2);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_launch_dependents();
  const uint32_t tZ1 = tmem_base;        // NZ buffers of 128 columns; W overlays part of each
  const uint32_t tZ2 = tmem_base + 256;
  const uint32_t tACC = tmem_base + 384;

  if (warp == 6) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      int bi = 0;    // ring items issued so far
      int kacc = 0;  // non-empty work items started so far
      auto put = [&](const CUtensorMap* map, int y, int bh) {
        const int slot = bi % NSLOT;
        const int use = bi / NSLOT;
        if (use > 0) ok = mbar_wait(&slot_empty[slot], (use - 1) & 1, ab, kFbSlotEmpty);
        if (!ok) return;
        mbar_expect_tx(&slot_full[slot], DB * BOX);
        for (int b = 0; b < DB; ++b) tma_load_3d(sRing + slot * ITEM + b * BOX, map, &slot_full[slot], b * 64, y, bh);
        ++bi;
      };
      for (int u = 0; u < n_steps && ok; ++u) {
        FaBwdItem it;
        if (!decode_step(u, it)) continue;
        if (it.n_iter == 0) continue;
        if (kacc > 0) ok = mbar_wait(r_free, (kacc - 1) & 1, ab, kFbRFree);
        if (!ok) break;
        mbar_expect_tx(r_full, Cfg::NR * Cfg::R_BYTES);
        for (int b = 0; b < DB; ++b) tma_load_3d(sR1 + b * BOX, &tmR1, r_full, b * 64, it.row0, it.bh);
        if (DUAL)
          for (int b = 0; b < DB; ++b) tma_load_3d(sR2 + b * BOX, &tmR2, r_full, b * 64, it.row0, it.bh);
        ++kacc;
        // consumption order: C1_0 (, C2_0); then for t >= 1: C1_t (, C2_t), T_{t-1}; finally T_{n-1}
        for (int t = 0; t <= it.n_iter && ok; ++t) {
          if (t < it.n_iter) {
            put(&tmC1, (it.t_start + t) * 128, it.bh);
            if (DUAL && ok) put(&tmC2, (it.t_start + t) * 128, it.bh);
          }
          if (t >= 1 && ok) put(&tmT, (it.t_start + t - 1) * 128, it.bh);
        }
      }
      if (!ok) {
        // abort path: let the copies already issued land before this CTA's shared memory is released
        if (kacc > 0) mbar_wait_drain(r_full, (kacc - 1) & 1, 2000000ull);
        for (int slot = 0; slot < NSLOT; ++slot)
          if (bi > slot) mbar_wait_drain(&slot_full[slot], ((bi - 1 - slot) / NSLOT) & 1, 2000000ull);
      }
    }
  } else if (warp == 4 || warp == 5) {
    // ------------------------------------------------------------------ MMA issuers (converged warps, one elected lane)
    // Ring positions inside a work item of n blocks (PER_BLOCK = NC + 1 items per block):
    //   C_t tile x:  t == 0 ? x : NC + (t-1) * PER_BLOCK + x ;   T_t:  NC + t * PER_BLOCK + (t + 1 < n ? NC : 0)
    constexpr uint32_t idesc_z = umma_idesc(128, 128, BF16, false, false);
    constexpr uint32_t idesc_acc = umma_idesc(128, DB == 2 ? 128 : 64, BF16, false, true);
    bool ok = true;
    int b0 = 0, g0 = 0, kacc = 0;
    const uint32_t r1_addr = smem_u32(sR1), r2_addr = smem_u32(sR2), ring_addr = smem_u32(sRing);
    for (int u = 0; u < n_steps && ok; ++u) {
      FaBwdItem it;
      if (!decode_step(u, it)) continue;
      const int n = it.n_iter;
      if (n == 0) continue;
      if (warp == 4) {
        ok = mbar_wait_warp(r_full, kacc & 1, ab, kFbR);
        for (int t = 0; t < n && ok; ++t) {
          const int g = g0 + t;
          if (g >= NZ) {
            ok = mbar_wait_warp(&z_free[g % NZ], (g / NZ - 1) & 1, ab, kFbZFree);
            if (!ok) break;
          }
          const int pos = b0 + (t == 0 ? 0 : NC + (t - 1) * PER_BLOCK);
          if (lane == 0) AB200_FBTR(1, g, 0);
          {
            const int slot = pos % NSLOT;
            ok = mbar_wait_warp(&slot_full[slot], (pos / NSLOT) & 1, ab, kFbSlotFull);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
              const uint32_t a = ring_addr + slot * ITEM;
              const uint32_t tz = tZ1 + (g % NZ) * 128;
#pragma unroll
              for (int b = 0; b < DB; ++b)
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                  umma_ss(tz, umma_smem_desc(r1_addr + b * BOX + ks * 32, 16, 1024),
                          umma_smem_desc(a + b * BOX + ks * 32, 16, 1024), idesc_z, (b > 0 || ks > 0) ? 1u : 0u);
              tc_commit(&slot_empty[slot]);
              tc_commit(&z_full[g % NZ]);
              if (!DUAL && t + 1 == n) tc_commit(r_free);
            }
            __syncwarp();
            if (lane == 0) AB200_FBTR(1, g, 1);
          }
          if (DUAL) {
            if (g >= 1) {
              // Z2 is single buffered: the element-wise threads must have read block g-1 out of it
              ok = mbar_wait_warp(z2_free, (g - 1) & 1, ab, kFbZ2Free);
              if (!ok) break;
            }
            if (lane == 0) AB200_FBTR(1, g, 2);
            const int slot = (pos + 1) % NSLOT;
            ok = mbar_wait_warp(&slot_full[slot], ((pos + 1) / NSLOT) & 1, ab, kFbSlotFull);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
              const uint32_t a = ring_addr + slot * ITEM;
#pragma unroll
              for (int b = 0; b < DB; ++b)
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                  umma_ss(tZ2, umma_smem_desc(r2_addr + b * BOX + ks * 32, 16, 1024),
                          umma_smem_desc(a + b * BOX + ks * 32, 16, 1024), idesc_z, (b > 0 || ks > 0) ? 1u : 0u);
              tc_commit(&slot_empty[slot]);
              tc_commit(z2_full);
              if (t + 1 == n) tc_commit(r_free);
            }
            __syncwarp();
            if (lane == 0) AB200_FBTR(1, g, 3);
          }
        }
      } else {
        for (int t = 0; t < n && ok; ++t) {
          const int g = g0 + t;
          if (t == 0 && kacc > 0) {
            ok = mbar_wait_warp(acc_free, (kacc - 1) & 1, ab, kFbAccFree);
            if (!ok) break;
          }
          ok = mbar_wait_warp(&w_full[g % NZ], (g / NZ) & 1, ab, kFbWFull);
          if (!ok) break;
          if (lane == 0) AB200_FBTR(1, g, 4);
          const int pos = b0 + NC + t * PER_BLOCK + (t + 1 < n ? NC : 0);
          const int slot = pos % NSLOT;
          ok = mbar_wait_warp(&slot_full[slot], (pos / NSLOT) & 1, ab, kFbSlotFull);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            const uint32_t a = ring_addr + slot * ITEM;
            const uint32_t tw = tZ1 + (g % NZ) * 128;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_ts(tACC, tw + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8), umma_smem_desc(a + ks * 2048, BOX, 1024), idesc_acc, (t > 0 || ks > 0) ? 1u : 0u);
            tc_commit(&slot_empty[slot]);
            tc_commit(&z_free[g % NZ]);
            if (t + 1 == n) tc_commit(acc_done);
          }
          __syncwarp();
          if (lane == 0) AB200_FBTR(1, g, 5);
        }
      }
      b0 += n * PER_BLOCK;
      g0 += n;
      ++kacc;
    }
  } else if (warp < 4 || (warp >= 8 && warp < 12)) {
    // ------------------------------------------------------------------ element-wise warpgroups
    // Group 0 (warps 0-3) handles columns 0-63 of every block, group 1 (warps 8-11) columns 64-127; thread `tid` of
    // either group owns TMEM lane (row) tid.
    const int grp = warp >> 3;
    const int tid = threadIdx.x & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    constexpr float kLog2e = 1.4426950408889634f;
    const uint64_t sl2 = f2_pack(p.scale * kLog2e, p.scale * kLog2e);
    const uint64_t sc2 = f2_pack(p.scale, p.scale);
    bool ok = true;
    int g0 = 0;
    for (int u = 0; u < n_steps && ok; ++u) {
      FaBwdItem it;
      if (!decode_step(u, it)) continue;
      const int bh = it.bh, row0 = it.row0, n_iter = it.n_iter;
      const int grow = row0 + tid;
      if (n_iter == 0) {
        // no block contributes to this tile: zeros (written, like every output of this kernel, only after the kernels
        // before it in the stream have completed: one of them may still be reading scratch data parked in `out`)
        pdl_grid_dependency_wait();
        if (grp == 0 && grow < rows_len) {
          uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * rows_len + grow) * D;
          for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      // per-row terms of the dQ kernel (rows are queries): -lse * log2(e) and -delta * scale
      float row_nl2 = 0.f, row_nds = 0.f;
      if (!ROWK) {
        const float delta = fa_bwd_delta_warp<D, BF16>(p.o, p.dout, bh, grow - lane, p.Lq, lane);
        if (grow < p.Lq) {
          row_nl2 = -p.lse[static_cast<size_t>(bh) * p.Lq + grow] * kLog2e;
          row_nds = LEAN ? -delta : -delta * p.scale;
        }
      }
      for (int t = 0; t < n_iter; ++t) {
        const int g = g0 + t;
        const int col0 = (it.t_start + t) * 128;
        // per-column terms of the dV / dK kernels (columns are queries), from the helper's table: the value of column
        // (chunk q, lane) sits in a register of that lane and travels by warp shuffle
        float col_nl2[2] = {0.f, 0.f}, col_nds[2] = {0.f, 0.f};
        if (threadIdx.x == 0) AB200_FBTR(0, g, 0);
        if (ROWK) {
          const int ts = g % Cfg::NTAB;
          ok = mbar_wait_warp(&tab_full[ts], (g / Cfg::NTAB) & 1, ab, kFbTabFull);
          if (!ok) break;
          const float* tab = ctab + ts * 256;
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            col_nl2[q] = tab[128 + (2 * grp + q) * 32 + lane];
            if (DUAL) col_nds[q] = tab[(2 * grp + q) * 32 + lane];
          }
          mbar_arrive(&tab_free[ts]);
        }
        const bool diag = p.causal && col0 == row0;  // the only block that straddles the diagonal (Lq == Lkv)
        if (threadIdx.x == 0) AB200_FBTR(0, g, 1);
        ok = mbar_wait_warp(&z_full[g % NZ], (g / NZ) & 1, ab, kFbZFull);
        if (!ok) break;
        if (threadIdx.x == 0) AB200_FBTR(0, g, 2);
        tc_fence_after();
        const uint32_t tz = tmem_addr(tZ1 + (g % NZ) * 128, lane_base, 0);
        const uint32_t tz2 = tmem_addr(tZ2, lane_base, 0);
        // Step 1, P = exp2(Z1 * scale * log2 e - lse * log2 e) for this thread's 64 columns, packed to 16 bits. The dV
        // kernel stores it as W; the others keep it in registers: this part runs while the second GEMM1 is still
        // in flight, and Z2 (single buffered) is then held only for a short multiply.
        auto prob2 = [&](uint32_t za, uint32_t zb, int q, int c, float& p0, float& p1) {
          const int chunk = 2 * grp + q;
          uint64_t nl2 = f2_pack(row_nl2, row_nl2);
          if (ROWK) nl2 = f2_pack(__shfl_sync(0xffffffffu, col_nl2[q], c), __shfl_sync(0xffffffffu, col_nl2[q], c + 1));
          float a0, a1;
          f2_unpack(ffma2(f2_pack(__uint_as_float(za), __uint_as_float(zb)), sl2, nl2), a0, a1);
          // AB200_FA_BWD_POLY=1 puts every other pair on the FMA pipes; measured at B=8 H=16 L=4096 d=128: 5.3-5.7 ms
          // per backward against 5.1-5.3 ms with all of them on the special-function unit (the step is bound by
          // instruction issue, not by that unit)
          if (AB200_FA_BWD_POLY && ((c >> 1) % AB200_FA_BWD_POLY_EVERY == 0)) {
            exp2_poly2(f2_pack(a0, a1), p0, p1);
          } else {
            p0 = ex2_approx(a0);
            p1 = ex2_approx(a1);
          }
          if (diag) {
            const int cc = chunk * 32 + c;  // column inside the block; the row inside the block is tid
            if (ROWK ? (cc < tid) : (cc > tid)) p0 = 0.f;
            if (ROWK ? (cc + 1 < tid) : (cc + 1 > tid)) p1 = 0.f;
          }
        };
        uint32_t pp[FUSED ? 1 : 32];
        if constexpr (!FUSED) {
          // both 32-column loads are issued before the wait: one exposed TMEM latency per block instead of two
          uint32_t z1[2][32];
          tmem_ld32(tz + (2 * grp) * 32, z1[0]);
          tmem_ld32(tz + (2 * grp + 1) * 32, z1[1]);
          tc_wait_ld();
#pragma unroll
          for (int q = 0; q < 2; ++q) {
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              float p0, p1;
              prob2(z1[q][c], z1[q][c + 1], q, c, p0, p1);
              pp[q * 16 + (c >> 1)] = pack2<BF16>(p0, p1);
            }
            if (!DUAL) tmem_st16(tz + grp * 64 + q * 16, &pp[q * 16]);
          }
        }
        if (DUAL) {
          // Step 2, dS = P .* (dP * scale - delta * scale)
          if (threadIdx.x == 0) AB200_FBTR(0, g, 3);
          ok = mbar_wait_warp(z2_full, g & 1, ab, kFbZ2Full);
          if (!ok) break;
          if (threadIdx.x == 0) AB200_FBTR(0, g, 4);
          tc_fence_after();
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int chunk = 2 * grp + q;
            uint32_t z2[32], z1[FUSED ? 32 : 1];
            tmem_ld32(tz2 + chunk * 32, z2);
            if constexpr (FUSED) tmem_ld32(tz + chunk * 32, z1);
            tc_wait_ld();
            if (q == 1) {
              // this thread's part of Z2 is in registers: the second GEMM1 of the next block may overwrite it
              tc_fence_before();
              mbar_arrive(z2_free);
              if (threadIdx.x == 0) AB200_FBTR(0, g, 5);
            }
            uint32_t pk[16];
#pragma unroll
            for (int c = 0; c < 32; c += 2) {
              uint64_t nds = f2_pack(row_nds, row_nds);
              if constexpr (LEAN) {
                float t0, t1;
                f2_unpack(fadd2(f2_pack(__uint_as_float(z2[c]), __uint_as_float(z2[c + 1])), nds), t0, t1);
                pk[c >> 1] = mul2_16<BF16>(pp[q * 16 + (c >> 1)], pack2<BF16>(t0, t1));
                continue;
              }
              if (ROWK) nds = f2_pack(__shfl_sync(0xffffffffu, col_nds[q], c), __shfl_sync(0xffffffffu, col_nds[q], c + 1));
              const uint64_t t2 = ffma2(f2_pack(__uint_as_float(z2[c]), __uint_as_float(z2[c + 1])), sc2, nds);
              uint64_t pr2;
              if constexpr (FUSED) {
                float p0, p1;
                prob2(z1[c], z1[c + 1], q, c, p0, p1);
                pr2 = f2_pack(p0, p1);
              } else {
                pr2 = fa_bwd_unpack2<BF16>(pp[q * 16 + (c >> 1)]);
              }
              float w0, w1;
              f2_unpack(fmul2(pr2, t2), w0, w1);
              pk[c >> 1] = pack2<BF16>(w0, w1);
            }
            tmem_st16(tz + grp * 64 + q * 16, pk);
          }
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&w_full[g % NZ]);
        if (threadIdx.x == 0) AB200_FBTR(0, g, 6);
      }
      if (!ok) break;
      g0 += n_iter;
    }
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ helper warpgroup: column tables and epilogue
    const int tid = threadIdx.x - 384;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    constexpr float kLog2e = 1.4426950408889634f;
    bool ok = true;
    int kacc = 0;
    // table cursor: runs ahead of the epilogue cursor by up to two blocks of the next work item
    int pu = 0, pt = 0, gp = 0;
    FaBwdItem pit;
    bool pvalid = false;
    int cache_bh = -1;
    uint32_t cache_valid = 0;  // bit b: block b of slice cache_bh is in dcache (each thread reads back only what it wrote)
    auto p_next_item = [&]() {
      pvalid = false;
      while (pu < n_steps) {
        const bool have = decode_step(pu, pit);
        ++pu;
        if (have && pit.n_iter > 0) {
          pvalid = true;
          pt = 0;
          return;
        }
      }
    };
    auto produce_one = [&]() -> bool {  // one block's table; false when there is nothing left (or on abort)
      if (!pvalid) return false;
      const int ts = gp % Cfg::NTAB;
      if (gp >= Cfg::NTAB) {
        ok = mbar_wait_warp(&tab_free[ts], ((gp / Cfg::NTAB) - 1) & 1, ab, kFbTabFree);
        if (!ok) return false;
      }
      if (tid == 0) AB200_FBTR(2, gp, 0);
      const int qi = (pit.t_start + pt) * 128 + tid;
      const size_t row = static_cast<size_t>(pit.bh) * p.Lq + qi;
      float* tab = ctab + ts * 256;
      // queries past the end: lse = +inf, i.e. P = 0
      tab[128 + tid] = (qi < p.Lq) ? -p.lse[row] * kLog2e : __int_as_float(0xff800000);
      if (DUAL) {
        const int qb = pit.t_start + pt;
        if (pit.bh != cache_bh) {
          cache_bh = pit.bh;
          cache_valid = 0;
        }
        float nds;
        if (qb < Cfg::DCACHE_BLOCKS && ((cache_valid >> qb) & 1u)) {
          nds = dcache[qb * 128 + tid];
        } else {
          nds = -fa_bwd_delta_warp<D, BF16>(p.o, p.dout, pit.bh, qi - lane, p.Lq, lane) * p.scale;
          if (qb < Cfg::DCACHE_BLOCKS) {
            dcache[qb * 128 + tid] = nds;
            cache_valid |= 1u << qb;
          }
        }
        tab[tid] = nds;
      }
      mbar_arrive(&tab_full[ts]);
      if (tid == 0) AB200_FBTR(2, gp, 1);
      ++gp;
      if (++pt == pit.n_iter) p_next_item();
      return true;
    };
    if (ROWK) p_next_item();
    int g_end = 0;  // blocks of the work items up to and including the one whose epilogue comes next
    for (int u = 0; u < n_steps && ok; ++u) {
      FaBwdItem it;
      if (!decode_step(u, it)) continue;
      if (it.n_iter == 0) continue;
      g_end += it.n_iter;
      if (ROWK) {
        while (ok && gp < g_end + 2 && produce_one()) {}
        if (!ok) break;
      }
      const int grow = it.row0 + tid;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(it.bh) * rows_len + grow) * D;
      ok = mbar_wait_warp(acc_done, kacc & 1, ab, kFbAccDone);
      if (!ok) break;
      tc_fence_after();
      // A programmatic dependent computes its first tile while its predecessor drains, but stores nothing before
      // that kernel has completed: the fused dK/dV kernel reads per-query terms parked in the dq buffer.
      if (kacc == 0) pdl_grid_dependency_wait();
      const uint32_t ta = tmem_addr(tACC, lane_base, 0);
      const float out_mul = LEAN ? p.scale : 1.f;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t rr[32];
        tmem_ld32(ta + c0, rr);
        tc_wait_ld();
        if (c0 + 32 >= D) {
          // the whole accumulator is in registers: GEMM2 of the next work item may overwrite it
          tc_fence_before();
          mbar_arrive(acc_free);
        }
        if (grow < rows_len) {
#pragma unroll
          for (int i = 0; i < 32; i += 16) {
            uint32_t v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              v[e] = pack2<BF16>(__uint_as_float(rr[i + 2 * e]) * out_mul, __uint_as_float(rr[i + 2 * e + 1]) * out_mul);
            st_global_v8(orow + c0 + i, v);
          }
        }
      }
      ++kacc;
    }
  }

  __syncwarp();
  // A programmatic dependent must not complete before the kernel it overlapped with.
  if (threadIdx.x == 0) pdl_grid_dependency_wait();
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
