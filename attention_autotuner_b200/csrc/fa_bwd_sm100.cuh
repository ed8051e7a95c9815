// Flash-attention backward for sm_100a as three kernels that each own their output tile (no atomics, no fp32
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
// memory: Z1 double buffered at columns [0,256), Z2 single at [256,384), ACC at [384,384+D). W (16-bit) overlays Z1:
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
  static constexpr int AUX_BYTES = NTAB * 1024 + 1024;  // tables, barriers, flags
  static constexpr int NSLOT_FIT = (232448 - 1024 - AUX_BYTES - NR * R_BYTES) / ITEM_BYTES;
  static constexpr int NSLOT = NSLOT_FIT > 5 ? 5 : NSLOT_FIT;
  static constexpr int SMEM_BYTES = 1024 + NR * R_BYTES + NSLOT * ITEM_BYTES + AUX_BYTES;
  static constexpr int NTHREADS = 512;
  static constexpr int TMEM_COLS = 512;
  static_assert(D == 64 || D == 128, "head dimension");
  static_assert(NSLOT >= 4, "ring too small");
};

// delta of one query row: sum_d dO[row,d] * O[row,d] (fp32 accumulation of 16-bit inputs)
template <int D, bool BF16>
__device__ __forceinline__ float fa_bwd_delta_row(const void* o, const void* dout, size_t row) {
  const uint4* po = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(o) + row * D);
  const uint4* pd = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(dout) + row * D);
  float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
  for (int i = 0; i < D / 8; ++i) {
    const uint4 a = __ldg(po + i), b = __ldg(pd + i);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
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
      s0 = fmaf(a0, b0, s0);
      s1 = fmaf(a1, b1, s1);
    }
  }
  return s0 + s1;
}

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
fa_bwd_sm100_kernel(const __grid_constant__ CUtensorMap tmR1, const __grid_constant__ CUtensorMap tmR2,
                    const __grid_constant__ CUtensorMap tmC1, const __grid_constant__ CUtensorMap tmC2,
                    const __grid_constant__ CUtensorMap tmT, const FaBwdParams p) {
  constexpr int D = Cfg::D, DB = Cfg::DB, NSLOT = Cfg::NSLOT, NC = Cfg::NC, ITEM = Cfg::ITEM_BYTES, BOX = Cfg::BOX_BYTES;
  constexpr bool DUAL = Cfg::DUAL, ROWK = Cfg::ROWK, BF16 = Cfg::BF16;
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
  uint64_t* z_full = slot_empty + NSLOT;      // [2] GEMM1 into Z1 buffer complete
  uint64_t* w_full = z_full + 2;              // [2] W written over the Z1 buffer (element-wise -> GEMM2)
  uint64_t* z_free = w_full + 2;              // [2] GEMM2 of a block complete: its Z1/W buffer may be rewritten
  uint64_t* z2_full = z_free + 2;             // [1] second GEMM1 complete
  uint64_t* z2_free = z2_full + 1;            // [1] Z2 read into registers (element-wise -> GEMM1 warp)
  uint64_t* acc_done = z2_free + 1;           // [1]
  uint64_t* acc_free = acc_done + 1;          // [1]
  uint64_t* r_free = acc_free + 1;            // [1]
  uint64_t* tab_full = r_free + 1;            // [NTAB] column table written            (helper -> element-wise)
  uint64_t* tab_free = tab_full + Cfg::NTAB;  // [NTAB] column table read into registers (element-wise -> helper)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tab_free + Cfg::NTAB);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 2);

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
  // Work list: pairs (k-th heaviest, k-th lightest row block of a slice) handed out round-robin, as in chain_sm100.cuh.
  const int npair = (p.nrb + 1) / 2;
  const int n_super = (p.total_items / p.nrb) * npair;
  const int n_steps = static_cast<int>(blockIdx.x) < n_super ? 2 * ((n_super - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
  auto decode_step = [&](int u, FaBwdItem& it) -> bool {
    const int sidx = blockIdx.x + gridDim.x * (u >> 1);
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
    for (int i = 0; i < 2; ++i) {
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
  const uint32_t tZ1 = tmem_base;        // two buffers of 128 columns; W overlays the first 64 of each
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
          if (g >= 2) {
            ok = mbar_wait_warp(&z_free[g & 1], ((g - 2) >> 1) & 1, ab, kFbZFree);
            if (!ok) break;
          }
          const int pos = b0 + (t == 0 ? 0 : NC + (t - 1) * PER_BLOCK);
          {
            const int slot = pos % NSLOT;
            ok = mbar_wait_warp(&slot_full[slot], (pos / NSLOT) & 1, ab, kFbSlotFull);
            if (!ok) break;
            tc_fence_after();
            if (elect_one()) {
              const uint32_t a = ring_addr + slot * ITEM;
              const uint32_t tz = tZ1 + (g & 1) * 128;
#pragma unroll
              for (int b = 0; b < DB; ++b)
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                  umma_ss(tz, umma_smem_desc(r1_addr + b * BOX + ks * 32, 16, 1024),
                          umma_smem_desc(a + b * BOX + ks * 32, 16, 1024), idesc_z, (b > 0 || ks > 0) ? 1u : 0u);
              tc_commit(&slot_empty[slot]);
              tc_commit(&z_full[g & 1]);
              if (!DUAL && t + 1 == n) tc_commit(r_free);
            }
            __syncwarp();
          }
          if (DUAL) {
            if (g >= 1) {
              // Z2 is single buffered: the element-wise threads must have read block g-1 out of it
              ok = mbar_wait_warp(z2_free, (g - 1) & 1, ab, kFbZ2Free);
              if (!ok) break;
            }
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
          }
        }
      } else {
        for (int t = 0; t < n && ok; ++t) {
          const int g = g0 + t;
          if (t == 0 && kacc > 0) {
            ok = mbar_wait_warp(acc_free, (kacc - 1) & 1, ab, kFbAccFree);
            if (!ok) break;
          }
          ok = mbar_wait_warp(&w_full[g & 1], (g >> 1) & 1, ab, kFbWFull);
          if (!ok) break;
          const int pos = b0 + NC + t * PER_BLOCK + (t + 1 < n ? NC : 0);
          const int slot = pos % NSLOT;
          ok = mbar_wait_warp(&slot_full[slot], (pos / NSLOT) & 1, ab, kFbSlotFull);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            const uint32_t a = ring_addr + slot * ITEM;
            const uint32_t tw = tZ1 + (g & 1) * 128;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_ts(tACC, tw + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8), umma_smem_desc(a + ks * 2048, BOX, 1024), idesc_acc, (t > 0 || ks > 0) ? 1u : 0u);
            tc_commit(&slot_empty[slot]);
            tc_commit(&z_free[g & 1]);
            if (t + 1 == n) tc_commit(acc_done);
          }
          __syncwarp();
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
        // no block contributes to this tile: zeros
        if (grp == 0 && grow < rows_len) {
          uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * rows_len + grow) * D;
          for (int c = 0; c < D; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      // per-row terms of the dQ kernel (rows are queries): -lse * log2(e) and -delta * scale
      float row_nl2 = 0.f, row_nds = 0.f;
      if (!ROWK && grow < p.Lq) {
        row_nl2 = -p.lse[static_cast<size_t>(bh) * p.Lq + grow] * kLog2e;
        row_nds = -fa_bwd_delta_row<D, BF16>(p.o, p.dout, static_cast<size_t>(bh) * p.Lq + grow) * p.scale;
      }
      for (int t = 0; t < n_iter; ++t) {
        const int g = g0 + t;
        const int col0 = (it.t_start + t) * 128;
        // per-column terms of the dV / dK kernels (columns are queries), from the helper's table: the value of column
        // (chunk q, lane) sits in a register of that lane and travels by warp shuffle
        float col_nl2[2] = {0.f, 0.f}, col_nds[2] = {0.f, 0.f};
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
        ok = mbar_wait_warp(&z_full[g & 1], (g >> 1) & 1, ab, kFbZFull);
        if (!ok) break;
        if (DUAL) {
          ok = mbar_wait_warp(z2_full, g & 1, ab, kFbZ2Full);
          if (!ok) break;
        }
        tc_fence_after();
        const uint32_t tz = tmem_addr(tZ1 + (g & 1) * 128, lane_base, 0);
        const uint32_t tz2 = tmem_addr(tZ2, lane_base, 0);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int chunk = 2 * grp + q;  // 32-column chunk of the block
          uint32_t z1[32], z2[32];
          tmem_ld32(tz + chunk * 32, z1);
          if (DUAL) tmem_ld32(tz2 + chunk * 32, z2);
          tc_wait_ld();
          if (DUAL && q == 1) {
            // this thread's part of Z2 is in registers: the second GEMM1 of the next block may overwrite it
            tc_fence_before();
            mbar_arrive(z2_free);
          }
          uint32_t pk[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            uint64_t nl2 = f2_pack(row_nl2, row_nl2), nds = f2_pack(row_nds, row_nds);
            if (ROWK) {
              nl2 = f2_pack(__shfl_sync(0xffffffffu, col_nl2[q], c), __shfl_sync(0xffffffffu, col_nl2[q], c + 1));
              if (DUAL) nds = f2_pack(__shfl_sync(0xffffffffu, col_nds[q], c), __shfl_sync(0xffffffffu, col_nds[q], c + 1));
            }
            float a0, a1;
            f2_unpack(ffma2(f2_pack(__uint_as_float(z1[c]), __uint_as_float(z1[c + 1])), sl2, nl2), a0, a1);
            float p0 = ex2_approx(a0), p1 = ex2_approx(a1);
            if (diag) {
              const int cc = chunk * 32 + c;  // column inside the block; the row inside the block is tid
              if (ROWK ? (cc < tid) : (cc > tid)) p0 = 0.f;
              if (ROWK ? (cc + 1 < tid) : (cc + 1 > tid)) p1 = 0.f;
            }
            if (DUAL) {
              // dS = P .* (dP * scale - delta * scale)
              const uint64_t t2 = ffma2(f2_pack(__uint_as_float(z2[c]), __uint_as_float(z2[c + 1])), sc2, nds);
              f2_unpack(fmul2(f2_pack(p0, p1), t2), p0, p1);
            }
            pk[c >> 1] = pack2<BF16>(p0, p1);
          }
          tmem_st16(tz + grp * 64 + q * 16, pk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&w_full[g & 1]);
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
      const int qi = (pit.t_start + pt) * 128 + tid;
      const size_t row = static_cast<size_t>(pit.bh) * p.Lq + qi;
      float* tab = ctab + ts * 256;
      // queries past the end: lse = +inf, i.e. P = 0
      tab[128 + tid] = (qi < p.Lq) ? -p.lse[row] * kLog2e : __int_as_float(0xff800000);
      if (DUAL) tab[tid] = (qi < p.Lq) ? -fa_bwd_delta_row<D, BF16>(p.o, p.dout, row) * p.scale : 0.f;
      mbar_arrive(&tab_full[ts]);
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
      const uint32_t ta = tmem_addr(tACC, lane_base, 0);
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
            for (int e = 0; e < 8; ++e) v[e] = pack2<BF16>(__uint_as_float(rr[i + 2 * e]), __uint_as_float(rr[i + 2 * e + 1]));
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
