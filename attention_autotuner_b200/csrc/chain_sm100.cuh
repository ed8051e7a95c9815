// Two-GEMM "chain" kernel for sm_100a, the common skeleton of the RetNet parallel forward and of the
// three kernels of its backward:
//
//     Z[128,128]  = R[128,K1] * C_t[128,K1]^T          (both operands K-major in shared memory)
//     W           = Z .* mask .* scale (./ r)           (registers; written back to TMEM as 16-bit)
//     ACC[128,N2] += W[128,128] * T_t[128,N2]           (W from tensor memory, T_t MN-major in smem)
//
// for t over the 128-wide blocks of the streamed ("column") side. R is the CTA's resident 128-row tile.
//
//   kernel   MODE   R (rows)    C_t         T_t            W                                 out
//   forward  Fwd    Q (query)   K block     V block chunk  S~ = QK^T*scale*M  (unnormalised)  O = ACC / max(sum|S~|,1), r
//   dV       RowK   K (key)     Q block     dO block chunk P^T = (S~)^T / r[query]            dV
//   dK       RowK   V (key)     dO block    Q block        G^T = (dO V^T)^T * M^T*scale/r     dK
//   dQ       RowQ   dO (query)  V block     K block        G   = (dO V^T) * M*scale/r         dQ
//
// These replace ret_fwd_regfuse / ret_fwd_smemfuse (csrc/kernels/retnet/regfuse/regfuse.h:47-459,
// csrc/kernels/retnet/smemfuse/smemfuse.h:62-635) and ret_bwd_colblock + convert_dq
// (csrc/kernels/retnet/bwd/bwd_colblock.h:81-811) of the reference. Differences by design:
//   * forward defers the normalisation: P stays unnormalised in 16-bit and O is divided by r once in the
//     epilogue (the reference rescales O every block, regfuse.h:296-316); fp16 P saturates instead of
//     overflowing;
//   * backward is three kernels that each own their output tile, so dQ needs neither fp32 atomics nor
//     the dq_accum scratch buffer nor a convert kernel (bwd_colblock.h:583-586, 742-811), and every
//     result is bit-reproducible;
//   * the mask is either the reference's general 16-bit tensor [H,Lq,Lkv] (read straight from L2 by
//     the thread that owns the row / column) or a per-head decay gamma, M[i,j] = gamma^(i-j) for i>=j,
//     computed in registers, with the all-zero blocks above the diagonal skipped.
//
// Roles: warps 0-3 element-wise warpgroup (thread t owns TMEM lane t), warp 4 issues GEMM1 and warp 5 GEMM2
// (converged warps, one elected lane each), warp 6 lane 0 is the TMA producer, warp 7 the scout that turns
// per-item ring arrivals into one arrival per operand tile, warps 8-11 the epilogue warpgroup. Z is double buffered in tensor
// memory so that GEMM1 of block t+1 runs while the warpgroup works on block t. All streamed operands
// travel through one ring of 32 KB items (two boxes of 128 rows x 64 columns, 128-byte swizzle).
#pragma once

#include "chain_common.cuh"

namespace ab200 {

template <int K1_, int N2_, int MODE_, bool GENERAL_, bool BF16_>
struct ChainConfig {
  static constexpr int K1 = K1_;      // contraction length of GEMM1 (multiple of 64, <= 512)
  static constexpr int N2 = N2_;      // accumulator columns per CTA (multiple of 64, <= 256)
  static constexpr int MODE = MODE_;
  static constexpr bool GENERAL = GENERAL_;
  static constexpr bool BF16 = BF16_;
  static constexpr int K1B = K1 / 64;  // boxes per C tile
  static constexpr int N2B = N2 / 64;  // boxes per T tile
  static constexpr int BOX_BYTES = 128 * 128;
  // A ring item is up to two boxes (32 KB): 128 columns of K for GEMM1, 128 columns of N for GEMM2, so that
  // every MMA is 128x128x16 (64 tensor-pipe cycles against ~49 cycles of issue cost per instruction).
  static constexpr int ITEM_BYTES = 2 * BOX_BYTES;
  static constexpr int CI = (K1B + 1) / 2;  // items per C tile
  static constexpr int TI = (N2B + 1) / 2;  // items per T tile
  static constexpr int R_BYTES = 128 * K1 * 2;
  static constexpr int AUX_BYTES = 2048;  // column-factor tables (2 x 128 floats), barriers, flags
  static constexpr int NSLOT_FIT = (232448 - 1024 - AUX_BYTES - R_BYTES) / ITEM_BYTES;
  static constexpr int NSLOT = NSLOT_FIT > 6 ? 6 : NSLOT_FIT;
  static constexpr int SMEM_BYTES = 1024 + R_BYTES + NSLOT * ITEM_BYTES + AUX_BYTES;
  static constexpr int NTHREADS = 384;  // element-wise warpgroup + {GEMM1, GEMM2, TMA producer, scout} + epilogue warpgroup
  static constexpr int TMEM_COLS = 512;  // 2 x 128 (Z) + N2
  static_assert(K1 % 64 == 0 && K1 >= 64 && K1 <= 512, "K1");
  static_assert(N2 % 64 == 0 && N2 >= 64 && N2 <= 256, "N2");
  static_assert(NSLOT >= 3, "ring too small");
  static_assert(2 * NSLOT + 20 <= 96, "barrier area");
};



template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
chain_sm100_kernel(const __grid_constant__ CUtensorMap tmR, const __grid_constant__ CUtensorMap tmC,
                   const __grid_constant__ CUtensorMap tmT, const ChainParams p) {
  constexpr int K1B = Cfg::K1B, N2B = Cfg::N2B, N2 = Cfg::N2, NSLOT = Cfg::NSLOT, MODE = Cfg::MODE;
  constexpr int CI = Cfg::CI, TI = Cfg::TI, ITEM = Cfg::ITEM_BYTES;
  constexpr bool GENERAL = Cfg::GENERAL, BF16 = Cfg::BF16;
  constexpr int BOX = Cfg::BOX_BYTES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sR = smem;
  uint8_t* sRing = smem + Cfg::R_BYTES;
  float* rs = reinterpret_cast<float*>(sRing + NSLOT * ITEM);  // [128] row sums of the finished item (forward)
  uint64_t* bars = reinterpret_cast<uint64_t*>(rs + 128);
  uint64_t* r_full = bars;                    // [1]
  uint64_t* slot_full = bars + 1;             // [NSLOT]
  uint64_t* slot_empty = slot_full + NSLOT;   // [NSLOT]
  uint64_t* z_full = slot_empty + NSLOT;      // [2]
  uint64_t* w_full = z_full + 2;              // [2]
  uint64_t* acc_done = w_full + 2;            // [1] GEMM2 of an item complete        (MMA -> element-wise)
  uint64_t* acc_free = acc_done + 1;          // [1] accumulator drained by the epilogue (element-wise -> MMA)
  uint64_t* r_free = acc_free + 1;            // [1] GEMM1 of an item complete: R may be overwritten (MMA -> TMA)
  uint64_t* z_free = r_free + 1;              // [2] GEMM2 of a block complete: its Z/W buffer may be rewritten
  uint64_t* c_ready = z_free + 2;             // [4] all ring items of a C tile have landed (scout -> GEMM1 warp)
  uint64_t* t_ready = c_ready + 4;            // [4] same for a T tile                      (scout -> GEMM2 warp)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(t_ready + 4);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
  const int lane = threadIdx.x & 31;
  // Persistent grid. Items are numbered  w = (bh * ny + chunk) * nrb + k,  row block = k-th heaviest, and taken in
  // an order (decode_step below) in which the CTAs running at any moment cover a few neighbouring slices
  // (operands shared in L2).
  // Loads, MMAs and element-wise work of consecutive items overlap: the producer prefetches the next item's
  // resident tile as soon as GEMM1 of the current one has finished (r_free), the epilogue of an item runs
  // while GEMM1 of the next one is already in flight, and only the first GEMM2 waits for it (acc_free).
  const int rows_len = (MODE == kChainRowK) ? p.Lkv : p.Lq;
  const int cols_len = (MODE == kChainRowK) ? p.Lq : p.Lkv;
  const int ncb = (cols_len + 127) / 128;
  auto decode = [&](int w) -> ChainItem {
    ChainItem it;
    const int k = w % p.nrb;
    const int rest = w / p.nrb;
    it.n_off = (rest % p.ny) * N2;
    it.bh = rest / p.ny;
    // heaviest row blocks first when blocks are skipped (Fwd/RowQ: late queries; RowK: early keys)
    const int rb = (p.skip_upper && MODE != kChainRowK) ? (p.nrb - 1 - k) : k;
    it.row0 = rb * 128;
    it.t_start = 0;
    it.n_iter = ncb;
    if (p.skip_upper) {
      if (MODE == kChainRowK) {
        it.t_start = rb;  // query blocks that end before this key block see none of its keys
        it.n_iter = ncb - rb;
      } else {
        it.n_iter = (rb + 1 < ncb) ? rb + 1 : ncb;  // key blocks up to the one holding the last query row
      }
      if (it.n_iter < 0) it.n_iter = 0;
    }
    return it;
  };
  // Work list of a CTA. With the blocks above the diagonal skipped the k-th heaviest and the k-th lightest row
  // block of a slice together always cost the same number of blocks, so the list is made of such pairs
  // ("super-items", heavy one first) and handed out round-robin: every CTA gets the same work up to one
  // super-item, whatever the grid size. Step u of a CTA: super-item blockIdx.x + gridDim.x * (u / 2), first or
  // second member.
  const int npair = (p.nrb + 1) / 2;
  const int n_super = (p.total_items / p.nrb) * npair;
  const int n_steps = static_cast<int>(blockIdx.x) < n_super ? 2 * ((n_super - blockIdx.x + gridDim.x - 1) / gridDim.x) : 0;
  auto decode_step = [&](int u, ChainItem& it) -> bool {
    const int sidx = blockIdx.x + gridDim.x * (u >> 1);
    const int j = sidx % npair;
    const int k = (u & 1) ? p.nrb - 1 - j : j;
    if ((u & 1) && k == j) return false;  // the middle row block of an odd count is its own partner
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
      mbar_init(&w_full[i], 128);
    }
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 128);
    mbar_init(r_free, 1);
    for (int i = 0; i < 2; ++i) mbar_init(&z_free[i], 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&c_ready[i], 1);
      mbar_init(&t_ready[i], 1);
    }
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 6 && lane == 0) {
    tma_prefetch_desc(&tmR);
    tma_prefetch_desc(&tmC);
    tma_prefetch_desc(&tmT);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  // The next kernel in the stream, if it was launched as a programmatic dependent (the backward's three kernels are
  // independent of each other), may take over SMs as this kernel's CTAs exit instead of waiting for the whole grid.
  pdl_launch_dependents();
  const uint32_t tZ0 = tmem_base;          // Z buffers at columns [0,128) and [128,256); W overlays the first 64
  const uint32_t tACC = tmem_base + 256;   // [256, 256+N2)

  // Register budget per role (setmaxnreg): the element-wise threads of the forward and of the mask-tensor flavours
  // need more than the 168 registers per thread that 384 threads get at launch. AB200_CHAIN_REBAL: 0 = never,
  // 1 = every flavour, 2 = only those flavours. Measured at config 4 in one session (forward + backward):
  // 1.244 / 1.225 / 1.40 ms for 0 / 1 / 2, so 1 is the default.
#ifndef AB200_CHAIN_REBAL
#define AB200_CHAIN_REBAL 1
#endif
  constexpr bool kRebalance = AB200_CHAIN_REBAL == 1 || (AB200_CHAIN_REBAL == 2 && ((MODE == kChainFwd) || GENERAL));
  if (warp >= 4 && warp < 8) {
  if constexpr (kRebalance) asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
  if (warp == 6) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      int bi = 0;    // ring items issued so far (all work items)
      int kacc = 0;  // non-empty work items started so far
      // one ring item = boxes [2i, 2i+2) of a tile (the last item of an odd tile holds one box)
      auto put = [&](const CUtensorMap* map, int x0, int nboxes, int y, int bh) {
        const int slot = bi % NSLOT;
        const int use = bi / NSLOT;
        if (use > 0) ok = mbar_wait(&slot_empty[slot], (use - 1) & 1, ab, kCtSlotEmpty);
        if (!ok) return;
        mbar_expect_tx(&slot_full[slot], nboxes * BOX);
        for (int b = 0; b < nboxes; ++b)
          tma_load_3d(sRing + slot * ITEM + b * BOX, map, &slot_full[slot], x0 + b * 64, y, bh);
        ++bi;
      };
      for (int u = 0; u < n_steps && ok; ++u) {
        ChainItem it;
        if (!decode_step(u, it)) continue;
        if (it.n_iter == 0) continue;
        // the resident tile may be overwritten once GEMM1 of the previous item has completed
        if (kacc > 0) ok = mbar_wait(r_free, (kacc - 1) & 1, ab, kCtRFree);
        if (!ok) break;
        mbar_expect_tx(r_full, Cfg::R_BYTES);
#pragma unroll
        for (int c = 0; c < K1B; ++c) tma_load_3d(sR + c * BOX, &tmR, r_full, c * 64, it.row0, it.bh);
        ++kacc;
        // consumption order: C_0, then for t >= 1: C_t, T_{t-1}; finally T_{n-1}
        for (int t = 0; t <= it.n_iter && ok; ++t) {
          if (t < it.n_iter) {
            for (int i = 0; i < CI && ok; ++i)
              put(&tmC, i * 128, (K1B - 2 * i) >= 2 ? 2 : 1, (it.t_start + t) * 128, it.bh);
          }
          if (t >= 1) {
            for (int i = 0; i < TI && ok; ++i)
              put(&tmT, it.n_off + i * 128, (N2B - 2 * i) >= 2 ? 2 : 1, (it.t_start + t - 1) * 128, it.bh);
          }
        }
      }
      if (!ok) {
        // abort path: let the copies already issued land before this CTA's shared memory is released
        if (kacc > 0) mbar_wait_drain(r_full, (kacc - 1) & 1, 2000000ull);
        for (int slot = 0; slot < NSLOT; ++slot)
          if (bi > slot) mbar_wait_drain(&slot_full[slot], ((bi - 1 - slot) / NSLOT) & 1, 2000000ull);
      }
    }
  } else if (warp == 7) {
    // ------------------------------------------------------------------ scout
    // Walks the ring in order, waits for every item to land and posts ONE arrival per operand tile
    // (c_ready / t_ready). The MMA warps then wait once per GEMM instead of once per ring item, and each ring
    // barrier keeps a single in-order waiter (two waiters on one parity-tracked barrier could alias phases).
    {
      bool ok = true;
      int bi = 0;
      int cg = 0, tg = 0;  // groups posted so far (a group = up to two ring items = up to 128 columns)
      auto post = [&](int nitems, uint64_t* ready, int& counter) {
        for (int i0 = 0; i0 < nitems && ok; i0 += 2) {
          for (int i = i0; i < nitems && i < i0 + 2 && ok; ++i, ++bi)
            ok = mbar_wait_warp(&slot_full[bi % NSLOT], (bi / NSLOT) & 1, ab, kCtSlotFull);
          if (ok && elect_one()) mbar_arrive(&ready[counter & 3]);
          __syncwarp();
          ++counter;
        }
      };
      for (int u = 0; u < n_steps && ok; ++u) {
        ChainItem it;
        if (!decode_step(u, it)) continue;
        const int n = it.n_iter;
        for (int t = 0; t <= n && ok && n > 0; ++t) {
          if (t < n) post(CI, c_ready, cg);
          if (t >= 1) post(TI, t_ready, tg);
        }
      }
    }
  } else if (warp == 4 || warp == 5) {
    // ------------------------------------------------------------------ MMA issuers
    // Warp 4 issues GEMM1 (Z), warp 5 issues GEMM2 (ACC). Measured on B200: the tensor pipe accepts only a
    // short queue of MMAs, so every barrier wait (~100 cycles even when already complete) and every commit
    // (~65 cycles) of a single issuing thread leaves the pipe idle; with two issuing warps the overhead of one
    // runs under the MMAs of the other. Each warp runs converged and one elected lane issues, so addresses and
    // descriptors stay warp-uniform. Ring items are consumed in a fixed order, so each warp computes the slots
    // of its own tiles:  C_0 at b0;  C_t at b0 + CI + (t-1)(CI+TI);  T_t right after C_{t+1}, except the last
    // T_{n-1}, which follows T_{n-2} directly.
    {
      constexpr uint32_t idesc_z = umma_idesc(128, 128, BF16, false, false);
      constexpr uint32_t idesc_acc2 = umma_idesc(128, 128, BF16, false, true);  // two boxes: N = 128
      constexpr uint32_t idesc_acc1 = umma_idesc(128, 64, BF16, false, true);   // one box:   N = 64
      bool ok = true;
      int b0 = 0;    // ring items of earlier work items
      int g0 = 0;    // 128-wide blocks of earlier work items (selects Z buffer and ready barrier)
      int kacc = 0;  // non-empty work items finished so far
      int cg = 0, tg = 0;  // operand groups consumed so far (as the scout counts them)
      const uint32_t r_addr = smem_u32(sR);
      const uint32_t ring_addr = smem_u32(sRing);
      for (int u = 0; u < n_steps && ok; ++u) {
        ChainItem it;
        if (!decode_step(u, it)) continue;
        const int n = it.n_iter;
        if (n == 0) continue;
        if (warp == 4) {
          ok = mbar_wait_warp(r_full, kacc & 1, ab, kCtR);
          for (int t = 0; t < n && ok; ++t) {
            const int g = g0 + t;
            if (g >= 2) {
              // Z buffer g&1 still holds W(g-2) until GEMM2 of block g-2 has read it
              ok = mbar_wait_warp(&z_free[g & 1], ((g - 2) >> 1) & 1, ab, kCtZFree);
              if (!ok) break;
            }
            if (lane == 0) AB200_CTR(1, g, 0);
            const uint32_t tz = tZ0 + (g & 1) * 128;
            const int base = b0 + (t == 0 ? 0 : CI + (t - 1) * (CI + TI));
#pragma unroll
            for (int i0 = 0; i0 < CI; i0 += 2) {
              ok = mbar_wait_warp(&c_ready[cg & 3], (cg >> 2) & 1, ab, kCtSlotFull);
              ++cg;
              if (!ok) break;
              tc_fence_after();
              if (elect_one()) {
#pragma unroll
                for (int i = i0; i < i0 + 2; ++i) {
                  if (i < CI) {
                    const int slot = (base + i) % NSLOT;
                    const uint32_t a = ring_addr + slot * ITEM;
                    const int nb = (K1B - 2 * i) >= 2 ? 2 : 1;
#pragma unroll
                    for (int b = 0; b < 2; ++b) {
                      if (b < nb) {
#pragma unroll
                        for (int ks = 0; ks < 4; ++ks)
                          umma_ss(tz, umma_smem_desc(r_addr + (2 * i + b) * BOX + ks * 32, 16, 1024),
                                  umma_smem_desc(a + b * BOX + ks * 32, 16, 1024), idesc_z,
                                  (i > 0 || b > 0 || ks > 0) ? 1u : 0u);
                      }
                    }
                    tc_commit(&slot_empty[slot]);
                  }
                }
                if (i0 + 2 >= CI) {
                  tc_commit(&z_full[g & 1]);
                  if (t + 1 == n) tc_commit(r_free);
                }
              }
              __syncwarp();
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) AB200_CTR(1, g, 1);
          }
        } else {
          for (int t = 0; t < n && ok; ++t) {
            const int g = g0 + t;
            if (t == 0 && kacc > 0) {
              // the first GEMM2 overwrites the accumulator: the previous item's epilogue must have read it
              ok = mbar_wait_warp(acc_free, (kacc - 1) & 1, ab, kCtAccFree);
              if (!ok) break;
            }
            ok = mbar_wait_warp(&w_full[g & 1], (g >> 1) & 1, ab, kCtWFull);
            if (!ok) break;
            if (lane == 0) AB200_CTR(1, g, 2);
            tc_fence_after();
            const uint32_t tw = tZ0 + (g & 1) * 128;
            const int base = b0 + CI + t * (CI + TI) + (t + 1 < n ? CI : 0);
#pragma unroll
            for (int i0 = 0; i0 < TI; i0 += 2) {
              ok = mbar_wait_warp(&t_ready[tg & 3], (tg >> 2) & 1, ab, kCtSlotFull);
              ++tg;
              if (!ok) break;
              tc_fence_after();
              if (elect_one()) {
#pragma unroll
                for (int i = i0; i < i0 + 2; ++i) {
                  if (i < TI) {
                    const int slot = (base + i) % NSLOT;
                    const uint32_t a = ring_addr + slot * ITEM;
                    const bool two = (N2B - 2 * i) >= 2;
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                      umma_ts(tACC + i * 128, tw + ks * 8, umma_smem_desc(a + ks * 2048, BOX, 1024),
                              two ? idesc_acc2 : idesc_acc1, (t > 0 || ks > 0) ? 1u : 0u);
                    tc_commit(&slot_empty[slot]);
                  }
                }
                if (i0 + 2 >= TI) {
                  tc_commit(&z_free[g & 1]);
                  if (t + 1 == n) tc_commit(acc_done);
                }
              }
              __syncwarp();
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) AB200_CTR(1, g, 3);
          }
        }
        b0 += n * (CI + TI);
        g0 += n;
        ++kacc;
      }
    }
  }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ element-wise warpgroup
    if constexpr (kRebalance) asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int tid = threadIdx.x;  // 0..127 = TMEM lane = row of the resident tile
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32);
    const bool decay_mode = !GENERAL;
    bool ok = true;
    int g0 = 0;     // blocks processed before the current work item
    int kacc = 0;   // non-empty work items finished so far

    for (int u = 0; u < n_steps && ok; ++u) {
      ChainItem it;
      if (!decode_step(u, it)) continue;
      const int bh = it.bh, row0 = it.row0, n_off = it.n_off, t_start = it.t_start, n_iter = it.n_iter;
      const int grow = row0 + tid;  // global row index on the row side
      const int h = bh % p.H;
      float lg = 0.f;  // log2(gamma)
      if (decay_mode) lg = log2f(p.decay[h]);
      // per-row factor that does not depend on the block
      float rowf_base = p.scale;
      if (decay_mode) rowf_base *= exp2f((MODE == kChainRowK ? -tid : tid) * lg);
      if (MODE == kChainRowQ) rowf_base *= (grow < p.Lq) ? 1.0f / p.r_in[static_cast<size_t>(bh) * p.Lq + grow] : 0.f;
      float rsum = 0.f;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * rows_len + grow) * p.ld_out + n_off;
      if (n_iter == 0) {
        // no block contributes to this tile: zeros (and r = 1 in the forward)
        if (grow < rows_len) {
          for (int c = 0; c < N2; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
          if (MODE == kChainFwd && n_off == 0) p.r_out[static_cast<size_t>(bh) * p.Lq + grow] = 1.0f;
        }
        continue;
      }

    for (int t = 0; t < n_iter; ++t) {
      const int g = g0 + t;  // running block index: Z buffer g & 1
      const int col0 = (t_start + t) * 128;
      float colf[4] = {0.f, 0.f, 0.f, 0.f};
      if (MODE == kChainRowK) {
        // gamma^c / r[c] (decay) or 1 / r[c] (mask tensor: lg = 0) of column (chunk, lane) in a register of that lane
#pragma unroll
        for (int q = 0; q < 4; ++q) colf[q] = chain_rowk_colf(p, bh, col0, q, lane, lg);
      }
      // mask tensor: this thread's 128 mask values of the block, packed in pairs, fetched before the wait for Z
      // (Fwd / RowQ: its row of the mask; RowK: its column, read by rows by the whole warp and transposed)
      uint32_t mk0[GENERAL ? 32 : 1], mk1[GENERAL ? 32 : 1];
      if constexpr (GENERAL && MODE != kChainRowK) {
        chain_mask_prefetch<MODE, 0>(p, h, grow, col0, mk0);
        chain_mask_prefetch<MODE, 2>(p, h, grow, col0, mk1);
      } else if constexpr (GENERAL) {
        if (p.mask_t != nullptr) {  // a transposed copy of the mask exists: the thread's column is a row of it
          chain_mask_prefetch_t<0>(p, h, grow, col0, mk0);
          chain_mask_prefetch_t<2>(p, h, grow, col0, mk1);
        } else {
          chain_mask_prefetch_rowk<0>(p, h, grow - lane, lane, col0, mk0);
          chain_mask_prefetch_rowk<2>(p, h, grow - lane, lane, col0, mk1);
        }
      }
      float rowf = rowf_base;
      if (decay_mode) rowf *= exp2f((MODE == kChainRowK ? (col0 - row0) : (row0 - col0)) * lg);
      // triangular predicate only on blocks that straddle the diagonal (decay mode)
      //   Fwd/RowQ: column c valid iff col0 + c <= grow ;  RowK: valid iff col0 + c >= grow
      const bool straddle = decay_mode && (MODE == kChainRowK ? (col0 < row0 + 127) : (col0 + 127 > row0));
      const int dlim = grow - col0;

      if (tid == 0) AB200_CTR(0, g, 0);
      ok = mbar_wait_warp(&z_full[g & 1], (g >> 1) & 1, ab, kCtZFull);
      if (!ok) break;
      if (tid == 0) AB200_CTR(0, g, 1);
      tc_fence_after();
      const uint32_t tz = tmem_addr(tZ0 + (g & 1) * 128, lane_base, 0);
      if constexpr (GENERAL) {
        chain_ew_mask2<MODE, BF16, 0, false>(tz, mk0, rowf, colf[0], colf[1], rsum);
        chain_ew_mask2<MODE, BF16, 2, false>(tz, mk1, rowf, colf[2], colf[3], rsum);
      } else {
        chain_ew_decay2<MODE, BF16, 0, false>(tz, rowf, lg, colf[0], colf[1], straddle, dlim, rsum);
        chain_ew_decay2<MODE, BF16, 2, false>(tz, rowf, lg, colf[2], colf[3], straddle, dlim, rsum);
      }
      if (MODE == kChainFwd && t + 1 == n_iter) {
        // hand the row sums to the epilogue warpgroup (single buffer: the previous item's epilogue, which
        // signals acc_free after reading it, must be through)
        if (kacc > 0) {
          ok = mbar_wait_warp(acc_free, (kacc - 1) & 1, ab, kCtAccFree);
          if (!ok) break;
        }
        rs[tid] = rsum;
      }
      if (tid == 0) AB200_CTR(0, g, 2);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&w_full[g & 1]);
      if (tid == 0) AB200_CTR(0, g, 3);
    }
      if (!ok) break;
      g0 += n_iter;
      ++kacc;
    }
  } else {
    // ------------------------------------------------------------------ epilogue warpgroup
    if constexpr (kRebalance) asm volatile("setmaxnreg.dec.sync.aligned.u32 112;");
    // Drains the accumulator of a finished work item (ACC -> scale -> 16-bit -> global) while the other roles
    // are already working on the next item; thread t owns TMEM lane t.
    const int tid = threadIdx.x - 256;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    bool ok = true;
    int kacc = 0;
    for (int u = 0; u < n_steps && ok; ++u) {
      ChainItem it;
      if (!decode_step(u, it)) continue;
      if (it.n_iter == 0) continue;  // the element-wise warpgroup writes the zeros of an empty tile
      const int grow = it.row0 + tid;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(it.bh) * rows_len + grow) * p.ld_out + it.n_off;
      ok = mbar_wait_warp(acc_done, kacc & 1, ab, kCtAccDone);
      if (!ok) break;
      tc_fence_after();
      float osc = 1.0f;
      if (MODE == kChainFwd) {
        const float r = fmaxf(rs[tid], 1.0f);
        osc = 1.0f / r;
        if (it.n_off == 0 && grow < rows_len) p.r_out[static_cast<size_t>(it.bh) * p.Lq + grow] = r;
      }
      const uint32_t ta = tmem_addr(tACC, lane_base, 0);
#pragma unroll
      for (int c0 = 0; c0 < N2; c0 += 32) {
        uint32_t rr[32];
        tmem_ld32(ta + c0, rr);
        tc_wait_ld();
        if (c0 + 32 >= N2) {
          // every column of the accumulator is in registers now: GEMM2 of the next item may overwrite it
          tc_fence_before();
          mbar_arrive(acc_free);
        }
        if (grow < rows_len) {
#pragma unroll
          for (int i = 0; i < 32; i += 16) {
            uint32_t v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              v[e] = pack2<BF16>(__uint_as_float(rr[i + 2 * e]) * osc, __uint_as_float(rr[i + 2 * e + 1]) * osc);
            st_global_v8(orow + c0 + i, v);
          }
        }
      }
      ++kacc;
    }
  }

  __syncwarp();
  // A programmatic dependent must not complete before the kernel it overlapped with: completion then stays
  // ordered along the stream for whatever comes next.
  if (threadIdx.x == 0) pdl_grid_dependency_wait();
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
