// Flash-attention backward for sm_100a: dK and dV of one 128-key tile in ONE kernel, so that S^T is computed once for
// both and every streamed tile of Q and dO is read once and used twice. Per block of 128 queries:
//
//     Z1[128 keys,128 q] = K Q_t^T   + X1 B_t^T      = S^T - lse[q] / scale                (SS MMAs, K = D + 16)
//     Z2[128 keys,128 q] = V dO_t^T  + X2 B_t^T      = dP^T - delta[q]                      (SS MMAs, K = D + 16)
//     W1 = P^T  = exp2(Z1 * scale * log2 e)                                                  (registers -> TMEM over Z1)
//     W2 = P^T .* Z2                                                                         (registers -> TMEM over Z2)
//     dV[128,D] += W1 dO_t          dK[128,D] += W2 Q_t     (TS MMAs; dK is multiplied by scale once, in the epilogue)
//
// The per-query terms (-lse / scale and -delta = -rowsum(dO .* O)) enter as one more K slice of the two first GEMMs: a
// constant operand X (column scales on the key side) times B_t, 128 rows of eight 16-bit values per query: each term
// is split into three 16-bit pieces whose weighted sum restores it to fp32 accuracy (fa_bwd_split3). The element-wise
// threads therefore need nothing per column: no table in shared memory, no shuffles. The pieces are computed once per
// call by fa_bwd_prep_kernel and parked in the dq buffer, which nobody else touches until the dQ kernel, the last of
// the backward, stores its first tile (it waits for this kernel to complete before that).
// The reference has no attention backward (python/ops/attention_interface.py:38-39 is `pass`); the formulas are the
// derivative of its forward (python/utils/ref_op.py:2-6) with the softmax recomputed from the forward's log-sum-exp.
//
// Z1 and Z2 are single buffered (tensor memory: Z1, Z2, dV and dK accumulators = 4 x 128 columns at D = 128), but the
// two chains S^T -> P^T -> dV and dP^T -> dS^T -> dK interleave, each issued by a warp of its own:
//     warp 4:  [dV += W1(t)[:, 0:64] dO_t[0:64]]  [dV += W1(t)[:, 64:128] dO_t[64:128] ; Z1(t+1)]
//     warp 5:  [dK += W2(t)[:, 0:64] Q_t[0:64]]   [dK += W2(t)[:, 64:128] Q_t[64:128] ; Z2(t+1)]
// The element-wise warps work P^T (two halves of 64 query columns), then dS^T (two halves), handing each half over as
// soon as it is written. The next block cannot start before its Z1, and the tensor core executes MMAs in the order
// they are issued, so warp 5 holds its last group back until warp 4 has issued Z1(t+1); that group then runs under
// the next block's exponentials.
// Roles (512 threads): warps 0-3 and 8-11 element-wise (two threads per key row),
// warps 4 and 5 MMA issue (one per chain), warp 6 lane 0 TMA producer, warps 12-15 epilogue (accumulators -> 16 bit -> global).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "fa_bwd_sm100.cuh"

namespace ab200 {

// Column scales of the three pieces. bf16 has the exponent range of fp32, so plain residuals do; fp16 pieces are
// spread over 2^8 ... 2^-12 so that values from 1e-9 to 1e7 keep 30 bits.
template <bool BF16>
struct FaBwdSplit {
  static constexpr float S0 = BF16 ? 1.f : 256.f;
  static constexpr float S1 = BF16 ? 1.f : 0.25f;
  static constexpr float S2 = BF16 ? 1.f : 0.000244140625f;  // 2^-12
};

template <bool BF16>
__device__ __forceinline__ uint16_t fa_bwd_to16(float x, float& back) {
  if constexpr (BF16) {
    const __nv_bfloat16 b = __float2bfloat16_rn(x);
    back = __bfloat162float(b);
    return __bfloat16_as_ushort(b);
  } else {
    const __half h = __float2half_rn(fminf(fmaxf(x, -65504.f), 65504.f));
    back = __half2float(h);
    return __half_as_ushort(h);
  }
}

// x ~= t[0] * S0 + t[1] * S1 + t[2] * S2 (greedy residuals; the scales are powers of two, so the residuals are exact).
template <bool BF16>
__device__ __forceinline__ void fa_bwd_split3(float x, uint16_t* t) {
  const float s[3] = {FaBwdSplit<BF16>::S0, FaBwdSplit<BF16>::S1, FaBwdSplit<BF16>::S2};
  if (!(fabsf(x) < 3.0e38f)) x = 0.f;
  float r = x;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    float back;
    t[i] = fa_bwd_to16<BF16>(r * (1.f / s[i]), back);
    r = fmaf(-back, s[i], r);
  }
}

// One block of 128 threads per 128 queries of a slice: the 16-byte row {lse pieces x3, delta pieces x3, 0, 0} of every
// query, rows past Lq zero, in the order [BH][nqb * 128].
template <int D, bool BF16>
__global__ void __launch_bounds__(128) fa_bwd_prep_kernel(const void* o, const void* dout, const float* lse, uint4* terms,
                                                          int Lq, int nqb, float scale) {
  const int bh = blockIdx.y, qb = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row0 = qb * 128 + warp * 32;
  const float delta = fa_bwd_delta_warp<D, BF16>(o, dout, bh, row0, Lq, lane);
  const int qi = row0 + lane;
  uint16_t t[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (qi < Lq) {
    fa_bwd_split3<BF16>(-lse[static_cast<size_t>(bh) * Lq + qi] / scale, t);
    fa_bwd_split3<BF16>(-delta, t + 3);
  }
  uint4 v;
  v.x = t[0] | (static_cast<uint32_t>(t[1]) << 16);
  v.y = t[2] | (static_cast<uint32_t>(t[3]) << 16);
  v.z = t[4] | (static_cast<uint32_t>(t[5]) << 16);
  v.w = 0;
  terms[(static_cast<size_t>(bh) * nqb + qb) * 128 + threadIdx.x] = v;
}

struct FaBwdKvParams {
  void* dk;            // [BH, Lkv, D] 16-bit
  void* dv;            // [BH, Lkv, D] 16-bit
  const uint4* terms;  // [BH, nqb * 128] rows of eight 16-bit values (fa_bwd_prep_kernel)
  int Lq, Lkv, nqb;
  float scale;
  int causal;          // 1: Lq == Lkv and key j > query i masked; query blocks before the key block are skipped
  int nrb;             // 128-key blocks
  int total_items;     // nrb * BH
};

enum FaBwdKvTag : int {
  kFkR = 51, kFkSlotFull = 52, kFkSlotEmpty = 53, kFkZ1Full = 54, kFkZ2Full = 55, kFkW1Full = 56, kFkW2Full = 57,
  kFkAccDone = 58, kFkAccFree = 59, kFkRFree = 60
};

template <int D_, bool BF16_>
struct FaBwdKvConfig {
  static constexpr int D = D_;
  static constexpr bool BF16 = BF16_;
  static constexpr int DB = D / 64;                    // 64-column boxes per tile
  static constexpr int BOX_BYTES = 128 * 128;
  static constexpr int ITEM_BYTES = DB * BOX_BYTES;    // one streamed tile (Q_t or dO_t)
  static constexpr int R_BYTES = 128 * D * 2;          // one resident tile (K or V)
  static constexpr int NSLOT = 4;                      // ring: items 2g (Q) and 2g + 1 (dO) of block g, two blocks deep
  static constexpr int NBX = NSLOT / 2;                // per-query term tiles, one per Q item in flight
  static constexpr int X_BYTES = 2048;                 // 128 rows x 8 values x 2 bytes
  static constexpr int X_REGION = (3 + NBX) * X_BYTES; // X1, X2, B ring, zeros
  static constexpr int SMEM_BYTES = 1024 + X_REGION + 2 * R_BYTES + NSLOT * ITEM_BYTES + 1024;
  static constexpr int NTHREADS = 512;
  static constexpr int TMEM_COLS = 512;
  static_assert(D == 64 || D == 128, "head dimension");
  static_assert(X_REGION % 1024 == 0, "the swizzled tiles behind the term tiles need 1024-byte alignment");
  static_assert(SMEM_BYTES <= 232448, "shared memory");
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
fa_bwd_kv_sm100_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                       const FaBwdKvParams p) {
  constexpr int D = Cfg::D, DB = Cfg::DB, NSLOT = Cfg::NSLOT, NBX = Cfg::NBX, ITEM = Cfg::ITEM_BYTES, BOX = Cfg::BOX_BYTES;
  constexpr int XB = Cfg::X_BYTES;
  constexpr bool BF16 = Cfg::BF16;
  // AB200_FA_BWD_KV_POLY=1: one column pair in AB200_FA_BWD_KV_POLY_EVERY takes its exponentials as a cubic on the
  // FMA pipes instead of the special-function unit
#ifndef AB200_FKV_MMA_UNROLL
#define AB200_FKV_MMA_UNROLL 16
#endif
  constexpr int MU = AB200_FKV_MMA_UNROLL;  // unroll factor of the MMA issue loops
#ifndef AB200_FA_BWD_KV_POLY
#define AB200_FA_BWD_KV_POLY 0
#endif
#ifndef AB200_FA_BWD_KV_POLY_EVERY
#define AB200_FA_BWD_KV_POLY_EVERY 2
#endif

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // term tiles (no swizzle, 8 K values per row; the other 8 of the MMA's K slice read the zero tile):
  //   [X1][X2][B ring: NBX][zeros]
  uint8_t* sX = smem;
  uint8_t* sR1 = smem + Cfg::X_REGION;  // K tile
  uint8_t* sR2 = sR1 + Cfg::R_BYTES;    // V tile
  uint8_t* sRing = sR2 + Cfg::R_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRing + NSLOT * ITEM);
  uint64_t* r_full = bars;                   // [1] K and V tiles landed
  uint64_t* r_free = bars + 1;               // [1] the last first-GEMMs of a work item are complete
  uint64_t* slot_full = bars + 2;            // [NSLOT]
  uint64_t* slot_empty = slot_full + NSLOT;  // [NSLOT]
  uint64_t* z1_full = slot_empty + NSLOT;    // [1]
  uint64_t* z2_full = z1_full + 1;           // [1]
  uint64_t* w1_full = z2_full + 1;           // [2] P^T of a half written over that half of Z1
  uint64_t* w2_full = w1_full + 2;           // [2] P^T .* Z2 of a half written over that half of Z2
  uint64_t* s_issued = w2_full + 2;          // [1] warp 4 has issued Z1 of the next block
  uint64_t* acc_done = s_issued + 1;         // [1]
  uint64_t* acc_free = acc_done + 1;         // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 2);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  const int ncb = (p.Lq + 127) / 128;
  auto decode = [&](int w) -> FaBwdItem {
    FaBwdItem it;
    const int rb = w % p.nrb;
    it.bh = w / p.nrb;
    it.row0 = rb * 128;
    it.t_start = 0;
    it.n_iter = ncb;
    if (p.causal) {
      it.t_start = rb;  // query blocks before this key block see none of its keys
      it.n_iter = ncb - rb;
      if (it.n_iter < 0) it.n_iter = 0;
    }
    return it;
  };
  // Work list: pairs (k-th heaviest, k-th lightest key block of a slice) handed out round-robin, so that under causal
  // masking every CTA gets the same number of blocks and neighbouring CTAs share a slice's operands in L2.
  const int npair = (p.nrb + 1) / 2;
  const int n_super = (p.total_items / p.nrb) * npair;
  const int n_steps = 2 * ((n_super + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x));
  auto decode_step = [&](int u, FaBwdItem& it) -> bool {
    const int sidx = (u >> 1) * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x);
    if (sidx >= n_super) return false;
    const int j = sidx % npair;
    const int k = (u & 1) ? p.nrb - 1 - j : j;
    if ((u & 1) && k == j) return false;
    it = decode((sidx / npair) * p.nrb + k);
    return true;
  };

  if (threadIdx.x == 0) {
    mbar_init(r_full, 1);
    mbar_init(r_free, 2);  // one commit from each of the two MMA warps
    for (int i = 0; i < NSLOT; ++i) {
      mbar_init(&slot_full[i], 1);
      mbar_init(&slot_empty[i], 2);  // every streamed tile is read by both MMA warps
    }
    mbar_init(z1_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&w1_full[i], 256);
      mbar_init(&w2_full[i], 256);
    }
    mbar_init(z2_full, 1);
    mbar_init(s_issued, 1);
    mbar_init(acc_done, 2);
    mbar_init(acc_free, 128);
    ab->flag = 0;
    fence_mbar_init();
  }
  {
    // X1: column scales at K positions 0-2 (the lse pieces), X2: at 3-5 (the delta pieces); every key row alike.
    // Row r of a term tile sits at (r / 8) * 128 + (r % 8) * 16 = r * 16.
    float back;
    const uint32_t s0 = fa_bwd_to16<BF16>(FaBwdSplit<BF16>::S0, back), s1 = fa_bwd_to16<BF16>(FaBwdSplit<BF16>::S1, back),
                   s2 = fa_bwd_to16<BF16>(FaBwdSplit<BF16>::S2, back);
    uint4* x = reinterpret_cast<uint4*>(sX);
    for (int i = threadIdx.x; i < Cfg::X_REGION / 16; i += Cfg::NTHREADS) {
      uint4 v = make_uint4(0, 0, 0, 0);
      if (i < 128) v = make_uint4(s0 | (s1 << 16), s2, 0, 0);
      else if (i < 256) v = make_uint4(0, s0 << 16, s1 | (s2 << 16), 0);
      x[i] = v;
    }
    fence_proxy_async_smem();
  }
  if (warp == 4) {
    tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 6 && lane == 0) {
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmDO);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  pdl_launch_dependents();
#ifdef AB200_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    g_fa_bwd_trace[2][0][0] = clock64();
    g_fa_bwd_trace[2][0][1] = static_cast<long long>(globaltimer_ns());
  }
#endif
  const uint32_t tZ1 = tmem_base;
  const uint32_t tZ2 = tmem_base + 128;
  const uint32_t tACCV = tmem_base + 256;
  const uint32_t tACCK = tmem_base + 384;

  if (warp == 6) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      int bi = 0;    // ring items issued so far (2 per block)
      int kacc = 0;  // non-empty work items started so far
      for (int u = 0; u < n_steps && ok; ++u) {
        FaBwdItem it;
        if (!decode_step(u, it)) continue;
        if (it.n_iter == 0) continue;
        if (kacc > 0) ok = mbar_wait(r_free, (kacc - 1) & 1, ab, kFkRFree);
        if (!ok) break;
        mbar_expect_tx(r_full, 2 * Cfg::R_BYTES);
        for (int b = 0; b < DB; ++b) tma_load_3d(sR1 + b * BOX, &tmK, r_full, b * 64, it.row0, it.bh);
        for (int b = 0; b < DB; ++b) tma_load_3d(sR2 + b * BOX, &tmV, r_full, b * 64, it.row0, it.bh);
        ++kacc;
        for (int t = 0; t < it.n_iter && ok; ++t) {
          const int qb = it.t_start + t;
          for (int which = 0; which < 2 && ok; ++which) {
            const int slot = bi % NSLOT;
            const int use = bi / NSLOT;
            if (use > 0) ok = mbar_wait(&slot_empty[slot], (use - 1) & 1, ab, kFkSlotEmpty);
            if (!ok) break;
            mbar_expect_tx(&slot_full[slot], DB * BOX + (which == 0 ? XB : 0));
            const CUtensorMap* map = which == 0 ? &tmQ : &tmDO;
            for (int b = 0; b < DB; ++b) tma_load_3d(sRing + slot * ITEM + b * BOX, map, &slot_full[slot], b * 64, qb * 128, it.bh);
            if (which == 0)
              bulk_load_1d(sX + (2 + slot / 2) * XB, p.terms + (static_cast<size_t>(it.bh) * p.nqb + qb) * 128, XB,
                           &slot_full[slot]);
            ++bi;
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
  } else if (warp == 4 || warp == 5) {
    // ------------------------------------------------------------------ MMA issuers (converged warps, one elected lane)
    // Warp 4 owns the chain S^T -> P^T -> dV (Z1, dV accumulator), warp 5 the chain dP^T -> dS^T -> dK (Z2, dK
    // accumulator): a tcgen05.mma costs its issuing thread about 50 cycles whatever its shape, and the 40 MMAs of a
    // block would keep one thread busy for as long as the tensor pipe needs to execute them.
    constexpr uint32_t idesc_z = umma_idesc(128, 128, BF16, false, false);
    constexpr uint32_t idesc_acc = umma_idesc(128, D, BF16, false, true);
    bool ok = true;
    int g0 = 0, kacc = 0, n_held = 0;
    const uint32_t r1_addr = smem_u32(sR1), r2_addr = smem_u32(sR2), ring_addr = smem_u32(sRing), x_addr = smem_u32(sX);
    const uint32_t zero_addr = x_addr + (2 + NBX) * XB;
    const uint64_t x1_desc = umma_smem_desc_noswizzle(x_addr, zero_addr - x_addr, 128);
    const uint64_t x2_desc = umma_smem_desc_noswizzle(x_addr + XB, zero_addr - (x_addr + XB), 128);
    // Descriptors are built once; an MMA's operand is its tile's descriptor plus a constant (the address field counts
    // 16-byte units and no tile crosses the 256 KB the field can hold), so that issuing an MMA costs two additions.
    const uint64_t d_r1 = umma_smem_desc(r1_addr, 16, 1024), d_r2 = umma_smem_desc(r2_addr, 16, 1024);
    const uint64_t d_ring_k = umma_smem_desc(ring_addr, 16, 1024);    // streamed tile as K-major B operand (first GEMMs)
    const uint64_t d_ring_mn = umma_smem_desc(ring_addr, BOX, 1024);  // streamed tile as MN-major B operand (second GEMMs)
    const uint64_t d_bx = umma_smem_desc_noswizzle(x_addr + 2 * XB, zero_addr - (x_addr + 2 * XB), 128);  // term tile 0
    auto wait_item = [&](int item) {
      ok = mbar_wait_warp(&slot_full[item % NSLOT], (item / NSLOT) & 1, ab, kFkSlotFull);
    };
    // K step j (16 queries) of half h of a W tile: the 32 values of queries h*64 ... +31 sit in columns
    // [h*64, h*64+16), those of queries h*64+32 ... +63 in [h*64+32, h*64+48) (each written by the group that read them)
    auto w_col = [](int h, int j) -> uint32_t { return static_cast<uint32_t>(h * 64 + (j < 2 ? j * 8 : 32 + (j - 2) * 8)); };
    // Z1 of global block g
    auto gemm1a = [&](int g, bool last_of_item, bool announce) {
      wait_item(2 * g);
      if (!ok) return;
      if (lane == 0) AB200_FBTR(1, g, 2);
      const int slot = (2 * g) % NSLOT;
      const uint64_t da = d_ring_k + ((slot * ITEM) >> 4);
      // the term tile landed with the Q item of this block; a tile further on moves the zero tile one tile closer
      const uint64_t dx = d_bx + (((g % NBX) * XB) >> 4) - (static_cast<uint64_t>(((g % NBX) * XB) >> 4) << 16);
      tc_fence_after();
      if (elect_one()) {
#pragma unroll MU
        for (int b = 0; b < DB; ++b)
#pragma unroll MU
          for (int ks = 0; ks < 4; ++ks)
            umma_ss(tZ1, d_r1 + ((b * BOX + ks * 32) >> 4), da + ((b * BOX + ks * 32) >> 4), idesc_z, (b > 0 || ks > 0) ? 1u : 0u);
        umma_ss(tZ1, x1_desc, dx, idesc_z, 1u);
        tc_commit(z1_full);
        tc_commit(&slot_empty[slot]);  // this warp's last use of the Q item (the other one: dK += W2 Q)
        if (last_of_item) tc_commit(r_free);
        if (announce) mbar_arrive(s_issued);
      }
      __syncwarp();
    };
    // dV += W1[half h] dO_t[rows of half h]
    auto gemm2a = [&](int g, int h, bool first_of_item, bool last_of_item) {
      ok = mbar_wait_warp(&w1_full[h], g & 1, ab, kFkW1Full);
      if (ok && h == 0) wait_item(2 * g + 1);
      if (!ok) return;
      if (lane == 0) AB200_FBTR(1, g, 4 + h);
      const int slot = (2 * g + 1) % NSLOT;
      const uint64_t da = d_ring_mn + ((slot * ITEM + h * 4 * 2048) >> 4);
      tc_fence_after();
      if (elect_one()) {
#pragma unroll MU
        for (int j = 0; j < 4; ++j)
          umma_ts(tACCV, tZ1 + w_col(h, j), da + ((j * 2048) >> 4), idesc_acc, (!first_of_item || h > 0 || j > 0) ? 1u : 0u);
        if (h == 1) {
          tc_commit(&slot_empty[slot]);  // this warp's last use of the dO item (the other one: Z2)
          if (last_of_item) tc_commit(acc_done);
        }
      }
      __syncwarp();
    };
    // Z2 of global block g
    auto gemm1b = [&](int g, bool last_of_item) {
      wait_item(2 * g);  // the term tile travels with the Q item
      if (ok) wait_item(2 * g + 1);
      if (!ok) return;
      const int slot = (2 * g + 1) % NSLOT;
      const uint64_t da = d_ring_k + ((slot * ITEM) >> 4);
      const uint64_t dx = d_bx + (((g % NBX) * XB) >> 4) - (static_cast<uint64_t>(((g % NBX) * XB) >> 4) << 16);
      tc_fence_after();
      if (elect_one()) {
#pragma unroll MU
        for (int b = 0; b < DB; ++b)
#pragma unroll MU
          for (int ks = 0; ks < 4; ++ks)
            umma_ss(tZ2, d_r2 + ((b * BOX + ks * 32) >> 4), da + ((b * BOX + ks * 32) >> 4), idesc_z, (b > 0 || ks > 0) ? 1u : 0u);
        umma_ss(tZ2, x2_desc, dx, idesc_z, 1u);
        tc_commit(z2_full);
        tc_commit(&slot_empty[slot]);
        if (last_of_item) tc_commit(r_free);
      }
      __syncwarp();
      if (lane == 0) AB200_FBTR(1, g, 7);
    };
    // dK += W2[half h] Q_t[rows of half h]
    auto gemm2b = [&](int g, int h, bool first_of_item, bool last_of_item) {
      ok = mbar_wait_warp(&w2_full[h], g & 1, ab, kFkW2Full);
      if (!ok) return;
      if (lane == 0) AB200_FBTR(1, g, 6);
      const int slot = (2 * g) % NSLOT;  // full: Z2 of this block waited for it
      const uint64_t da = d_ring_mn + ((slot * ITEM + h * 4 * 2048) >> 4);
      tc_fence_after();
      if (elect_one()) {
#pragma unroll MU
        for (int j = 0; j < 4; ++j)
          umma_ts(tACCK, tZ2 + w_col(h, j), da + ((j * 2048) >> 4), idesc_acc, (!first_of_item || h > 0 || j > 0) ? 1u : 0u);
        if (h == 1) {
          tc_commit(&slot_empty[slot]);
          if (last_of_item) tc_commit(acc_done);
        }
      }
      __syncwarp();
    };
    for (int u = 0; u < n_steps && ok; ++u) {
      FaBwdItem it;
      if (!decode_step(u, it)) continue;
      const int n = it.n_iter;
      if (n == 0) continue;
      ok = mbar_wait_warp(r_full, kacc & 1, ab, kFkR);
      if (!ok) break;
      if (warp == 4) {
        gemm1a(g0, n == 1, false);
      } else {
        gemm1b(g0, n == 1);
      }
      for (int t = 0; t < n && ok; ++t) {
        const int g = g0 + t;
        if (t == 0 && kacc > 0) {
          ok = mbar_wait_warp(acc_free, (kacc - 1) & 1, ab, kFkAccFree);
          if (!ok) break;
        }
        if (warp == 4) {
          // the first half of the dV MMAs runs while the element-wise warps still work on the second half of P^T;
          // Z1 is free again as soon as the MMAs that read W1 are issued (MMAs execute in order)
          gemm2a(g, 0, t == 0, t + 1 == n);
          if (ok) gemm2a(g, 1, t == 0, t + 1 == n);
          if (ok && t + 1 < n) gemm1a(g + 1, t + 2 == n, true);
        } else {
          // The MMAs of this chain can run under the next block's exponentials; those of the other chain cannot (P^T of
          // the next block needs its Z1), and the tensor core takes MMAs in the order they are issued: so this warp
          // lets Z1 of the next block complete first. (With a ring of two blocks the barrier cannot run a whole
          // phase ahead of this wait: Z1 of block g + 2 needs the Q slot that the MMAs below release.)
          gemm2b(g, 0, t == 0, t + 1 == n);
          // The tensor core takes MMAs in the order they are issued. What is left of this chain can run under the next
          // block's exponentials; Z1 of the next block cannot: this warp lets warp 4 issue it first.
          if (ok && t + 1 < n) {
            ok = mbar_wait_warp(&w2_full[1], g & 1, ab, kFkW2Full);
            if (ok) ok = mbar_wait_warp(s_issued, n_held & 1, ab, kFkZ1Full);
            ++n_held;
          }
          if (ok) gemm2b(g, 1, t == 0, t + 1 == n);
          if (ok && t + 1 < n) gemm1b(g + 1, t + 2 == n);
        }
      }
      g0 += n;
      ++kacc;
    }
  } else if (warp < 4 || (warp >= 8 && warp < 12)) {
    // ------------------------------------------------------------------ element-wise warpgroups
    // A block is worked in two halves of 64 query columns; of each half, group 0 (warps 0-3) takes the first 32 columns
    // and group 1 (warps 8-11) the other 32; thread `tid` of either group owns TMEM lane (key row) tid. The 16-bit
    // results go over the first 16 of the 32 accumulator columns their thread read.
    const int grp = warp >> 3;
    const int tid = threadIdx.x & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    constexpr float kLog2e = 1.4426950408889634f;
    const uint64_t sl2 = f2_pack(p.scale * kLog2e, p.scale * kLog2e);
    bool ok = true;
    int g0 = 0;
    for (int u = 0; u < n_steps && ok; ++u) {
      FaBwdItem it;
      if (!decode_step(u, it)) continue;
      const int row0 = it.row0, n_iter = it.n_iter;
      if (n_iter == 0) {
        // no query block contributes to this key tile: zeros
        const int grow = row0 + tid;
        if (grp == 0 && grow < p.Lkv) {
          const size_t off = (static_cast<size_t>(it.bh) * p.Lkv + grow) * D;
          uint16_t* r1 = reinterpret_cast<uint16_t*>(p.dk) + off;
          uint16_t* r2 = reinterpret_cast<uint16_t*>(p.dv) + off;
          for (int c = 0; c < D; c += 8) {
            *reinterpret_cast<uint4*>(r1 + c) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(r2 + c) = make_uint4(0, 0, 0, 0);
          }
        }
        continue;
      }
      for (int t = 0; t < n_iter; ++t) {
        const int g = g0 + t;
        const bool diag = p.causal && (it.t_start + t) * 128 == row0;  // the only block that straddles the diagonal
        const uint32_t tz1 = tmem_addr(tZ1, lane_base, grp * 32);
        const uint32_t tz2 = tmem_addr(tZ2, lane_base, grp * 32);
        if (threadIdx.x == 0) AB200_FBTR(0, g, 0);
        uint32_t pp[32];  // this thread's 2 x 32 values of P^T, packed
        ok = mbar_wait_warp(z1_full, g & 1, ab, kFkZ1Full);
        if (!ok) break;
        if (threadIdx.x == 0) AB200_FBTR(0, g, 1);
        tc_fence_after();
        // P^T first, both halves (the chain S^T -> P^T -> dV -> next S^T is the one the next block waits for) ...
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t z[32];
          tmem_ld32(tz1 + h * 64, z);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            const uint64_t a2 = fmul2(f2_pack(__uint_as_float(z[c]), __uint_as_float(z[c + 1])), sl2);
            float p0, p1;
            if (AB200_FA_BWD_KV_POLY && ((c >> 1) % AB200_FA_BWD_KV_POLY_EVERY == 0)) {
              exp2_poly2(a2, p0, p1);
            } else {
              float a0, a1;
              f2_unpack(a2, a0, a1);
              p0 = ex2_approx(a0);
              p1 = ex2_approx(a1);
            }
            if (diag) {
              const int cc = h * 64 + grp * 32 + c;  // query inside the block; the key inside the block is tid
              if (cc < tid) p0 = 0.f;
              if (cc + 1 < tid) p1 = 0.f;
            }
            pp[h * 16 + (c >> 1)] = pack2<BF16>(p0, p1);
          }
          tmem_st16(tz1 + h * 64, &pp[h * 16]);
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(&w1_full[h]);
          if (threadIdx.x == 0) AB200_FBTR(0, g, 2 + h);
        }
        // ... then dS^T, both halves
        ok = mbar_wait_warp(z2_full, g & 1, ab, kFkZ2Full);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t z[32], pk[16];
          tmem_ld32(tz2 + h * 64, z);
          tc_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 2)
            pk[c >> 1] = mul2_16<BF16>(pp[h * 16 + (c >> 1)], pack2<BF16>(__uint_as_float(z[c]), __uint_as_float(z[c + 1])));
          tmem_st16(tz2 + h * 64, pk);
          tc_wait_st();
          tc_fence_before();
          mbar_arrive(&w2_full[h]);
          if (threadIdx.x == 0) AB200_FBTR(0, g, 4 + h);
        }
        if (!ok) break;
      }
      if (!ok) break;
      g0 += n_iter;
    }
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ epilogue warpgroup
    const int tid = threadIdx.x - 384;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    bool ok = true;
    int kacc = 0;
    for (int u = 0; u < n_steps && ok; ++u) {
      FaBwdItem it;
      if (!decode_step(u, it)) continue;
      if (it.n_iter == 0) continue;
      const int grow = it.row0 + tid;
      const size_t off = (static_cast<size_t>(it.bh) * p.Lkv + grow) * D;
      ok = mbar_wait_warp(acc_done, kacc & 1, ab, kFkAccDone);
      if (!ok) break;
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t ta = tmem_addr(which == 0 ? tACCV : tACCK, lane_base, 0);
        uint16_t* orow = reinterpret_cast<uint16_t*>(which == 0 ? p.dv : p.dk) + off;
        const float mul = which == 0 ? 1.f : p.scale;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t rr[32];
          tmem_ld32(ta + c0, rr);
          tc_wait_ld();
          if (which == 1 && c0 + 32 >= D) {
            // both accumulators are in registers: the second GEMMs of the next work item may overwrite them
            tc_fence_before();
            mbar_arrive(acc_free);
          }
          if (grow < p.Lkv) {
#pragma unroll
            for (int i = 0; i < 32; i += 16) {
              uint32_t v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                v[e] = pack2<BF16>(__uint_as_float(rr[i + 2 * e]) * mul, __uint_as_float(rr[i + 2 * e + 1]) * mul);
              st_global_v8(orow + c0 + i, v);
            }
          }
        }
      }
      ++kacc;
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
#ifdef AB200_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    g_fa_bwd_trace[2][0][2] = clock64();
    g_fa_bwd_trace[2][0][3] = static_cast<long long>(globaltimer_ns());
  }
#endif
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
