// flash-attention forward for sm_100a, persistent form of fa_fwd_sm100_kernel (same tile, same roles, same
// arithmetic): a grid of one CTA per SM walks a static work list instead of one CTA per 256 query rows.
//
// What the non-persistent kernel pays per CTA -- launch, tensor-memory allocation, barrier set-up, the Q load, the
// first S = Q K^T before any softmax can start, and at the end a last P V and an epilogue under which nothing else
// runs -- is about 3.4 KV blocks' worth of time (measured through the causal case, whose CTAs average 16.5 blocks
// at L = 4096 instead of 32, and through longer sequences). Here tensor memory and barriers live for the whole
// kernel; the Q tiles of the next work item are loaded as soon as the last S MMA of the current one has read them;
// the MMA warp goes straight from the last P V of one item to the first S of the next, so one query tile's epilogue
// (tensor memory -> registers -> global) runs under the other tile's GEMMs and under its own next S.
//
// Work list: items are (slice, V-column chunk, block of 256 query rows). Pairs of items of equal total cost (k-th
// heaviest and k-th lightest query block of a slice under a causal mask) are handed out round-robin, so every CTA
// gets the same work up to one pair, and neighbouring CTAs work on the same slice (K and V shared in L2).
// Replaces the reference kernels flashattn_fwd_regfuse (csrc/kernels/attention/regfuse/regfuse.h:48-455) and
// flashattn_fwd_smemfuse (csrc/kernels/attention/smemfuse/smemfuse.h:61-614), like fa_fwd_sm100.cuh.
#pragma once

#include "fa_fwd_sm100.cuh"

namespace ab200 {

enum FaPersistTag : int { kTagQFree = 8, kTagOFree = 9 };

struct FaFwdPersistParams {
  FaFwdParams f;
  int nqb;      // blocks of 256 query rows per slice
  int ndv;      // V-column chunks
  int n_super;  // pairs of work items: BH * ndv * ceil(nqb / 2)
};

struct FaFwdItem {
  int bh, dv_off, m_base;
  int nblk[2];
  int nmax;
};

// Output staging: where shared memory has room for both finished tiles (a K / V ring of up to three entries at
// d = 128), a tile's rows are written there (16-bit, 128-byte swizzle) and leave through TMA stores, one per warp and
// 64-column box (32 rows each, so no warp waits for another). A thread storing its own row writes 32-byte pieces of 32
// different rows per instruction, which keeps the softmax warps from the next item's first block for as long as a
// couple of KV blocks take.
template <class Cfg>
struct FaFwdPersistLayout {
  static constexpr int O_TILE_BYTES = Cfg::BM * Cfg::DV * 2;
#ifdef AB200_FA_FWD_NO_STAGE_O  // build option for comparisons: every thread stores its own row
  static constexpr bool STAGE_O = false;
#else
  static constexpr bool STAGE_O = Cfg::DV % 64 == 0 && Cfg::SMEM_BYTES + 2 * O_TILE_BYTES <= 232448;
#endif
  static constexpr int SMEM_BYTES = Cfg::SMEM_BYTES + (STAGE_O ? 2 * O_TILE_BYTES : 0);
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
fa_fwd_persist_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                            const FaFwdPersistParams pp) {
  static_assert(Cfg::NQ == 2 && Cfg::SPLIT == 1 && Cfg::NMMA == 1 && Cfg::EXP_EMU == 0 && Cfg::EXP_H2 == 0,
                "the persistent kernel is built for the default tile only");
  static_assert(Cfg::DV <= 128, "the epilogue holds a whole output row in registers");
  constexpr int DQK = Cfg::DQK, DV = Cfg::DV, NQ = 2, NSTAGE = Cfg::NSTAGE;
  constexpr bool BF16 = Cfg::BF16;
  constexpr int BM = Cfg::BM, BN = Cfg::BN;
  const FaFwdParams& p = pp.f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + NQ * Cfg::Q_TILE_BYTES;
  using Lay = FaFwdPersistLayout<Cfg>;
  constexpr bool STAGE_O = Lay::STAGE_O;
  uint8_t* sO = smem + Cfg::SMEM_TILES;  // [2] finished tiles on their way out (STAGE_O only)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::SMEM_TILES + (STAGE_O ? 2 * Lay::O_TILE_BYTES : 0));
  uint64_t* q_full = bars;                   // [2] Q tile landed
  uint64_t* q_free = q_full + NQ;            // [2] the item's last S MMA of the tile is complete
  uint64_t* kv_full = q_free + NQ;           // [NSTAGE]
  uint64_t* kv_empty = kv_full + NSTAGE;     // [NSTAGE]
  uint64_t* s_full = kv_empty + NSTAGE;      // [2]
  uint64_t* p_full = s_full + NQ;            // [2]
  uint64_t* o_done = p_full + NQ;            // [2]
  uint64_t* o_free = o_done + NQ;            // [2] the finished tile's O is in the softmax threads' registers
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(o_free + NQ);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);
  static_assert((4 * NQ + 2 * NSTAGE + 4 * NQ) * 8 + 16 <= 256, "barrier area");

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  constexpr int kMmaWarp = 4 * NQ;
  constexpr int kTmaWarp = 4 * NQ + 1;

  const int nblk_all = (p.Lkv + BN - 1) / BN;
  const int npair = (pp.nqb + 1) / 2;
  const int n_steps = 2 * ((pp.n_super + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x));
  // u-th work item of this CTA; false if there is none at this position
  auto get_item = [&](int u, FaFwdItem& it) -> bool {
    const int sidx = (u >> 1) * static_cast<int>(gridDim.x) + static_cast<int>(blockIdx.x);
    if (sidx >= pp.n_super) return false;
    const int j = sidx % npair;
    // heavy block first: under a causal mask the late query blocks see the most keys
    const int qb = (u & 1) ? j : pp.nqb - 1 - j;
    if ((u & 1) && qb == pp.nqb - 1 - j) return false;  // odd number of blocks: the middle one is alone
    const int sl = sidx / npair;
    it.bh = sl / pp.ndv;
    it.dv_off = (sl % pp.ndv) * DV;
    it.m_base = qb * (BM * NQ);
    it.nmax = 0;
#pragma unroll
    for (int s = 0; s < NQ; ++s) {
      int n = nblk_all;
      if (p.causal) {
        const int last_col = it.m_base + s * BM + (BM - 1) + (p.Lkv - p.Lq);
        const int nc = last_col < 0 ? 0 : last_col / BN + 1;
        n = nc < n ? nc : n;
      }
      if (it.m_base + s * BM >= p.Lq) n = 0;  // tile entirely past the end of Q
      it.nblk[s] = n;
      it.nmax = n > it.nmax ? n : it.nmax;
    }
    return true;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < NQ; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_free[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_done[i], 1);
      mbar_init(&o_free[i], 128);
    }
    for (int i = 0; i < NSTAGE; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == kTmaWarp && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp >= kMmaWarp) {
    // 384 threads start with 168 registers each; the softmax threads take 208 (a 128-column score row), which
    // leaves this warpgroup 88: 256 x 208 + 128 x 88 = 384 x 168. (setmaxnreg.inc waits, with no limit, until the
    // registers it asks for have been released: the two numbers must add up to no more than the CTA was given.)
    static_assert(256 * 208 + 128 * 88 <= 384 * 168, "register split of the warpgroups");
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    if (warp == kTmaWarp) {
      // ------------------------------------------------------------------ TMA producer
      if (lane == 0) {
        bool ok = true;
        int t = 0;                 // ring items issued so far (all work items)
        int nq_loaded[NQ] = {0, 0};
        for (int u = 0; u < n_steps && ok; ++u) {
          FaFwdItem it;
          if (!get_item(u, it)) continue;
          auto load_q = [&](int s) {
            if (it.nblk[s] == 0 || !ok) return;
            // the tile's buffer is free once the previous item's last S MMA of this tile has read it
            if (nq_loaded[s] > 0) ok = mbar_wait(&q_free[s], (nq_loaded[s] - 1) & 1, ab, kTagQFree);
            if (!ok) return;
            mbar_expect_tx(&q_full[s], Cfg::Q_TILE_BYTES);
#pragma unroll
            for (int c = 0; c < DQK / 64; ++c)
              tma_load_3d(sQ + s * Cfg::Q_TILE_BYTES + c * (BM * 128), &tmQ, &q_full[s], c * 64, it.m_base + s * BM, it.bh);
            ++nq_loaded[s];
          };
          load_q(0);
          // ring items of this work item: 2j = K block j, 2j+1 = V block j
          for (int i = 0; i < 2 * it.nmax && ok; ++i, ++t) {
            const int slot = t % NSTAGE;
            const int use = t / NSTAGE;
            if (use > 0) ok = mbar_wait(&kv_empty[slot], (use - 1) & 1, ab, kTagKvEmpty);
            if (!ok) break;
            uint8_t* dst = sKV + slot * Cfg::KV_SLOT_BYTES;
            const int j = i >> 1;
            if ((i & 1) == 0) {
              mbar_expect_tx(&kv_full[slot], Cfg::K_TILE_BYTES);
#pragma unroll
              for (int c = 0; c < DQK / 64; ++c) tma_load_3d(dst + c * (BN * 128), &tmK, &kv_full[slot], c * 64, j * BN, it.bh);
            } else {
              mbar_expect_tx(&kv_full[slot], Cfg::V_TILE_BYTES);
#pragma unroll
              for (int c = 0; c < DV / 64; ++c)
                tma_load_3d(dst + c * (BN * 128), &tmV, &kv_full[slot], it.dv_off + c * 64, j * BN, it.bh);
            }
            if (i == 0) load_q(1);
          }
        }
        if (!ok) {
          // abort path: let the copies already issued land before this CTA's shared memory is released
          for (int s = 0; s < NQ; ++s)
            if (nq_loaded[s] > 0) mbar_wait_drain(&q_full[s], (nq_loaded[s] - 1) & 1, 2000000ull);
          for (int slot = 0; slot < NSTAGE; ++slot)
            if (t > slot) mbar_wait_drain(&kv_full[slot], ((t - 1 - slot) / NSTAGE) & 1, 2000000ull);
        }
      }
    } else if (warp == kMmaWarp) {
      // ------------------------------------------------------------------ MMA issuer (converged warp, one elected lane)
      constexpr uint32_t idesc_qk = umma_idesc(BM, BN, BF16, false, false);
      constexpr uint32_t idesc_pv = umma_idesc(BM, DV, BF16, false, true);
      bool ok = true;
      int t0 = 0;           // ring items of the work items before the current one
      int full_waited = 0;  // ring items (global count) whose kv_full has been waited for
      int n_items[NQ] = {0, 0};   // work items with at least one block, per tile, before the current one
      int blk_done[NQ] = {0, 0};  // blocks of the tile in those items (phase base of p_full)
      auto wait_item = [&](int t) -> bool {
        while (ok && full_waited <= t) {
          ok = mbar_wait_warp(&kv_full[full_waited % NSTAGE], (full_waited / NSTAGE) & 1, ab, kTagKvFull);
          ++full_waited;
        }
        return ok;
      };
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t kv_addr = smem_u32(sKV);
      for (int u = 0; u < n_steps && ok; ++u) {
        FaFwdItem it;
        if (!get_item(u, it)) continue;
        // S_s = Q_s K_j^T; releases the K slot if this tile is its last user, the Q tile after the tile's last block
        auto issue_s = [&](int s, int j, bool release) {
          const int slot = (t0 + 2 * j) % NSTAGE;
          const uint32_t qa = q_addr + s * Cfg::Q_TILE_BYTES;
          const uint32_t ka = kv_addr + slot * Cfg::KV_SLOT_BYTES;
          const bool last_s = (j + 1 == it.nblk[s]);
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < DQK / 16; ++ks) {
              const uint32_t off = (ks >> 2) * (BM * 128) + (ks & 3) * 32;
              umma_ss(tmem_base + s * 128, umma_smem_desc(qa + off, 16, 1024), umma_smem_desc(ka + off, 16, 1024),
                      idesc_qk, ks > 0 ? 1u : 0u);
            }
            tc_commit(&s_full[s]);
            if (release) tc_commit(&kv_empty[slot]);
            if (last_s) tc_commit(&q_free[s]);
          }
          __syncwarp();
        };
        // O_s += P_s V_j; releases the V slot if this tile is its last user
        auto issue_pv = [&](int s, int j, bool release) {
          const int slot = (t0 + 2 * j + 1) % NSTAGE;
          const uint32_t va = kv_addr + slot * Cfg::KV_SLOT_BYTES;
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < BN / 16; ++ks)
              umma_ts(tmem_base + NQ * 128 + s * DV, tmem_base + s * 128 + ks * 8,
                      umma_smem_desc(va + ks * 2048, BN * 128, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
            tc_commit(&o_done[s]);
            if (release) tc_commit(&kv_empty[slot]);
          }
          __syncwarp();
        };
        int last_user = -1;
#pragma unroll
        for (int s = 0; s < NQ; ++s)
          if (it.nblk[s] > 0) last_user = s;
        // prologue: S_s(0). The S columns of the tile are free: the last P V of the previous item has been issued.
#pragma unroll
        for (int s = 0; s < NQ; ++s) {
          if (it.nblk[s] > 0 && ok) {
            ok = mbar_wait_warp(&q_full[s], n_items[s] & 1, ab, kTagQ);
            if (ok && wait_item(t0)) {
              tc_fence_after();
              issue_s(s, 0, s == last_user);
            }
          }
        }
        for (int j = 0; j < it.nmax && ok; ++j) {
          // users of V_j are the tiles with nblk > j; users of K_{j+1} those with nblk > j+1
          int last_v = -1, last_k = -1;
#pragma unroll
          for (int s = 0; s < NQ; ++s) {
            if (it.nblk[s] > j) last_v = s;
            if (it.nblk[s] > j + 1) last_k = s;
          }
#pragma unroll
          for (int s = 0; s < NQ; ++s) {
            if (it.nblk[s] > j && ok) {
              if (!wait_item(t0 + 2 * j + 1)) break;
              if (j == 0 && n_items[s] > 0) {
                // the first P V of an item overwrites O: the previous item's epilogue must have read it
                ok = mbar_wait_warp(&o_free[s], (n_items[s] - 1) & 1, ab, kTagOFree);
                if (!ok) break;
              }
              // p_full of this tile completes once per block; blocks of earlier items are counted in its phase
              ok = mbar_wait_warp(&p_full[s], (blk_done[s] + j) & 1, ab, kTagPFull);
              if (!ok) break;
              tc_fence_after();
              issue_pv(s, j, s == last_v);
            }
            if (it.nblk[s] > j + 1 && ok) {
              if (!wait_item(t0 + 2 * j + 2)) break;
              tc_fence_after();
              issue_s(s, j + 1, s == last_k);
            }
          }
        }
        t0 += 2 * it.nmax;
#pragma unroll
        for (int s = 0; s < NQ; ++s) {
          if (it.nblk[s] > 0) ++n_items[s];
          blk_done[s] += it.nblk[s];
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int s = warp >> 2;                    // query tile of this warpgroup
    const int row_in_tile = threadIdx.x & 127;  // TMEM lane
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    const uint32_t tS = tmem_addr(tmem_base, lane_base, s * 128);
    const uint32_t tO = tmem_addr(tmem_base, lane_base, NQ * 128 + s * DV);
    const int causal_shift = p.Lkv - p.Lq;
    bool ok = true;
    int cs = 0;  // blocks of this tile in the work items before the current one (phase base of s_full / o_done)
    for (int u = 0; u < n_steps && ok; ++u) {
      FaFwdItem it;
      if (!get_item(u, it)) continue;
      const int n_my = s == 0 ? it.nblk[0] : it.nblk[1];  // (a select: indexing by s would put the item in local memory)
      const int row = it.m_base + s * BM + row_in_tile;
      // (the output address is formed where it is used: a 64-bit value less to keep across the block loop)
      // and the item is decoded again for it: only the tile's row and block count stay live across the block loop)
      const int m_tile = it.m_base + s * BM;
      auto out_row = [&]() -> uint16_t* {
        FaFwdItem io;
        get_item(u, io);
        return reinterpret_cast<uint16_t*>(p.o) + (static_cast<size_t>(io.bh) * p.Lq + row) * p.dv_total + io.dv_off;
      };
      auto lse_row = [&]() -> float* {
        FaFwdItem io;
        get_item(u, io);
        return (p.lse != nullptr && io.dv_off == 0) ? p.lse + static_cast<size_t>(io.bh) * p.Lq + row : nullptr;
      };
      if (n_my == 0) {
        uint16_t* orow = out_row();
        // no visible key at all for this tile (causal with Lkv < Lq), or the tile lies past the end of Q
        if (row < p.Lq) {
          for (int c = 0; c < DV; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
          if (float* l = lse_row()) *l = -INFINITY;
        }
        continue;
      }
      float m_ref = -INFINITY;  // reference maximum (raw score units) the exponentials are taken against
      float l_sum = 0.f;        // running sum of exp
      for (int j = 0; j < n_my; ++j) {
        ok = mbar_wait_warp(&s_full[s], (cs + j) & 1, ab, kTagSFull);
        if (!ok) break;
        tc_fence_after();
        float sv[BN];
        {
          uint32_t* r = reinterpret_cast<uint32_t*>(sv);
          tmem_ld32(tS + 0, r + 0);
          tmem_ld32(tS + 32, r + 32);
          tmem_ld32(tS + 64, r + 64);
          tmem_ld32(tS + 96, r + 96);
          tc_wait_ld();
        }
        const int n0 = j * BN;
        // masking: keys past Lkv (ragged tail) and, under causal, keys j > i + shift
        const bool tail_blk = (n0 + BN > p.Lkv);
        const bool diag_blk = p.causal && (n0 + BN - 1 > m_tile + causal_shift);
        if (tail_blk || diag_blk) {
          int limit = p.Lkv - n0;  // columns [limit, BN) are masked
          if (p.causal) {
            const int cl = row + causal_shift - n0 + 1;
            limit = cl < limit ? cl : limit;
          }
#pragma unroll
          for (int c = 0; c < BN; ++c)
            if (c >= limit) sv[c] = -INFINITY;
        }
        // row maximum: four independent chains of three-input maxima
        float mA = sv[0], mB = sv[1], mC = sv[2], mD = sv[3];
#pragma unroll
        for (int c = 4; c < BN - 4; c += 8) {
          mA = fmax3(mA, sv[c], sv[c + 1]);
          mB = fmax3(mB, sv[c + 2], sv[c + 3]);
          mC = fmax3(mC, sv[c + 4], sv[c + 5]);
          mD = fmax3(mD, sv[c + 6], sv[c + 7]);
        }
        mA = fmax3(mA, sv[BN - 4], sv[BN - 3]);
        mB = fmax3(mB, sv[BN - 2], sv[BN - 1]);
        const float m_blk = fmaxf(fmaxf(mA, mB), fmaxf(mC, mD));

        // Lazy rescale: keep the old reference unless the maximum grew by more than 2^8 in the exp2 domain.
        bool need = (j == 0) || ((m_blk - m_ref) * p.scale_log2 > Cfg::RESCALE_LOG2);
        if (m_blk == -INFINITY) need = false;
        if (__any_sync(0xffffffffu, need)) {
          float alpha = 1.0f;
          if (need) {
            alpha = (m_ref == -INFINITY) ? 0.0f : ex2_approx((m_ref - m_blk) * p.scale_log2);
            m_ref = m_blk;
            l_sum *= alpha;
          }
          if (j > 0) {
            // O of this tile was last written by PV(j-1): wait for it, then scale the rows in place.
            ok = mbar_wait_warp(&o_done[s], (cs + j - 1) & 1, ab, kTagODone);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < DV; c0 += 32) {
              uint32_t r[32];
              tmem_ld32(tO + c0, r);
              tc_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
              tmem_st32(tO + c0, r);
            }
          }
        }
        const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref * p.scale_log2;
        // P = exp2(S * scale_log2 - m * scale_log2): packed FMA, MUFU ex2, four packed partial sums
        const uint64_t sl2 = f2_pack(p.scale_log2, p.scale_log2);
        const uint64_t nm2 = f2_pack(neg_m, neg_m);
        uint64_t acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t pk[BN / 4];
#pragma unroll
          for (int c = 0; c < BN / 2; c += 2) {
            const int cc = h * (BN / 2) + c;
            float x0, x1;
            f2_unpack(ffma2(f2_pack(sv[cc], sv[cc + 1]), sl2, nm2), x0, x1);
            const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
            acc[(c >> 1) & 3] = fadd2(acc[(c >> 1) & 3], f2_pack(e0, e1));
            pk[c >> 1] = pack2<BF16>(e0, e1);
          }
          tmem_st32(tS + h * (BN / 4), pk);
        }
        {
          float a0, a1;
          f2_unpack(fadd2(fadd2(acc[0], acc[1]), fadd2(acc[2], acc[3])), a0, a1);
          l_sum += a0 + a1;
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[s]);
      }
      if (!ok) break;
      // epilogue: O / l -> global, lse. O goes to registers first so that the next item's first P V may overwrite it.
      ok = mbar_wait_warp(&o_done[s], (cs + n_my - 1) & 1, ab, kTagODone);
      if (!ok) break;
      tc_fence_after();
      const float inv_l = l_sum > 0.f ? 1.0f / l_sum : 0.f;
      {
        uint16_t* orow = out_row();
        uint32_t r[DV];
#pragma unroll
        for (int c0 = 0; c0 < DV; c0 += 32) tmem_ld32(tO + c0, r + c0);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(&o_free[s]);
        if constexpr (STAGE_O) {
          (void)orow;
          // this warp's stores of the previous item must have read the staging rows before they are written again
          if (lane == 0) tma_store_wait_read0();
          __syncwarp();
          uint8_t* stage = sO + s * Lay::O_TILE_BYTES + row_in_tile * 128;
#pragma unroll
          for (int i = 0; i < DV; i += 8) {
            uint4 v;
            v.x = pack2<BF16>(__uint_as_float(r[i + 0]) * inv_l, __uint_as_float(r[i + 1]) * inv_l);
            v.y = pack2<BF16>(__uint_as_float(r[i + 2]) * inv_l, __uint_as_float(r[i + 3]) * inv_l);
            v.z = pack2<BF16>(__uint_as_float(r[i + 4]) * inv_l, __uint_as_float(r[i + 5]) * inv_l);
            v.w = pack2<BF16>(__uint_as_float(r[i + 6]) * inv_l, __uint_as_float(r[i + 7]) * inv_l);
            const int chunk16 = (i & 63) >> 3;
            *reinterpret_cast<uint4*>(stage + (i >> 6) * (BM * 128) + ((chunk16 ^ (row_in_tile & 7)) << 4)) = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            FaFwdItem io;
            get_item(u, io);
            const int row0 = m_tile + (warp & 3) * 32;
            if (row0 < p.Lq) {  // rows past the end of Q are clipped by the store
#pragma unroll
              for (int b = 0; b < DV / 64; ++b)
                tma_store_3d(&tmO, sO + s * Lay::O_TILE_BYTES + b * (BM * 128) + (warp & 3) * (32 * 128), io.dv_off + b * 64, row0,
                             io.bh);
              tma_store_commit();
            }
          }
        } else if (row < p.Lq) {
#pragma unroll
          for (int i = 0; i < DV; i += 16) {
            uint32_t v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              v[e] = pack2<BF16>(__uint_as_float(r[i + 2 * e]) * inv_l, __uint_as_float(r[i + 2 * e + 1]) * inv_l);
            st_global_v8(orow + i, v);
          }
        }
      }
      if (row < p.Lq)
        if (float* l = lse_row()) *l = (l_sum > 0.f) ? (m_ref * p.scale + __logf(l_sum)) : -INFINITY;
      cs += n_my;
    }
    if (STAGE_O && lane == 0) tma_store_wait0();  // all output written before the CTA's shared memory is released
  }

  // common tail: every role gets here, also after an aborted wait
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
