// Flash-attention forward on CTA pairs (cta_group::2): a cluster of two CTAs on the two SMs of a TPC owns 512 query
// rows of one (batch, head) slice, 256 per CTA as two ping-ponging tiles of 128 (as fa_fwd_sm100_kernel). Every MMA
// spans both CTAs (M = 256: tile s of the leader and tile s of the peer), issued by the leader's MMA warp:
//     S_s = Q_s K_j^T   each CTA holds its Q tiles and 64 of the 128 keys of K_j       (SS, B split by rows)
//     O_s += P_s V_j    P in each CTA's tensor memory, each CTA holds half of V_j's columns (TS, B split by columns)
// so each SM streams half of K and V from L2 and, above all, reads 6 KB instead of 8 KB of shared memory per S MMA:
// the single-CTA kernel's S GEMM (128 x 128 x 16: 4 KB of Q + 4 KB of K per 64 tensor cycles) needs the whole
// shared-memory bandwidth of its SM; with the softmax arithmetic removed that kernel still only reaches 77 % of
// the cuBLAS rate.
//
// Roles per CTA: warps 0-3 / 4-7 softmax of tile 0 / 1 (thread = row), warp 8 MMA issuer (leader CTA only; allocates
// tensor memory in both), warp 9 TMA producer (own Q tiles, own halves of K and V), warp 10 scout (relays "my half
// landed" to the leader's barriers), warp 11 idle. Completions of MMAs go to both CTAs with one tcgen05.commit each;
// no copy is broadcast across the cluster.
#pragma once

#include "fa_fwd_sm100.cuh"
#include "ptx_pair.cuh"

namespace ab200 {

template <int DQK_, int NSTAGE_, bool BF16_>
struct FaPairConfig {
  static constexpr int DQK = DQK_;        // head dim of Q/K, multiple of 64
  static constexpr int DV = 128;          // V columns per pair (tensor memory: 2 x 128 S + 2 x 128 O = 512 columns)
  static constexpr int NQ = 2;
  static constexpr int NSTAGE = NSTAGE_;  // K/V ring depth (half tiles)
  static constexpr bool BF16 = BF16_;
  static constexpr int BM = 128;
  static constexpr int BN = 128;
  static constexpr int NTHREADS = 384;
  static constexpr int Q_TILE_BYTES = BM * DQK * 2;
  static constexpr int K_HALF_BYTES = (BN / 2) * DQK * 2;   // 64 keys x DQK
  static constexpr int V_HALF_BYTES = BN * (DV / 2) * 2;    // 128 keys x 64 columns
  static constexpr int KV_SLOT_BYTES = K_HALF_BYTES > V_HALF_BYTES ? K_HALF_BYTES : V_HALF_BYTES;
  static constexpr int TMEM_COLS = 512;
  static constexpr int SMEM_TILES = NQ * Q_TILE_BYTES + NSTAGE * KV_SLOT_BYTES;
  static constexpr int SMEM_BYTES = SMEM_TILES + 1024 /*alignment slack*/ + 512 /*barriers*/;
  static_assert(DQK % 64 == 0 && DQK <= 256, "head dim");
  static_assert((5 * NQ + 3 * NSTAGE) * 8 + 16 <= 512, "barrier area");
  static_assert(SMEM_BYTES <= 232448, "shared memory overflow");
};

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::NTHREADS, 1)
fa_fwd_pair_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const FaFwdParams p) {
  constexpr int DQK = Cfg::DQK, DV = Cfg::DV, NQ = Cfg::NQ, NSTAGE = Cfg::NSTAGE;
  constexpr bool BF16 = Cfg::BF16;
  constexpr int BM = Cfg::BM, BN = Cfg::BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + NQ * Cfg::Q_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::SMEM_TILES);
  // "own": each CTA uses its copy for its own data; "leader": only the leader's copy, both CTAs arrive on it
  uint64_t* q_full = bars;                   // own    [NQ] Q tile landed (transaction count)
  uint64_t* kv_full = q_full + NQ;           // own    [NSTAGE] half tile landed
  uint64_t* kv_empty = kv_full + NSTAGE;     // own    [NSTAGE] MMAs that read the slot completed (commit from the leader)
  uint64_t* s_full = kv_empty + NSTAGE;      // own    [NQ] S_s complete
  uint64_t* o_done = s_full + NQ;            // own    [NQ] O_s += P_s V_j complete
  uint64_t* p_full = o_done + NQ;            // leader [NQ] P_s written by the 256 softmax threads of the pair
  uint64_t* q_ready = p_full + NQ;           // leader [NQ] Q tile s of both CTAs landed (2 arrivals)
  uint64_t* kv_ready = q_ready + NQ;         // leader [NSTAGE] both halves of a ring item landed (2 arrivals)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(kv_ready + NSTAGE);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
  const int lane = threadIdx.x & 31;
  constexpr int kMmaWarp = 8, kTmaWarp = 9, kScoutWarp = 10;
  const uint32_t rank = cluster_ctarank();

  // grid: x = 2 * (512-row query blocks), y = V-column chunk, z = (batch, head). Heaviest (latest) query blocks
  // first under a causal mask.
  const int n_qblk = gridDim.x >> 1;
  const int qblk = p.causal ? (n_qblk - 1 - (blockIdx.x >> 1)) : (blockIdx.x >> 1);
  const int bh = blockIdx.z;
  const int dv_off = blockIdx.y * DV;
  const int m_base = qblk * (2 * NQ * BM) + static_cast<int>(rank) * (NQ * BM);  // first query row of this CTA

  // KV blocks a tile needs (causal: up to the block holding its last visible key); every MMA spans both CTAs, so
  // tile s of both runs through the larger of the two counts and masks the surplus blocks completely.
  const int nblk_all = (p.Lkv + BN - 1) / BN;
  auto need = [&](int r, int s) -> int {
    const int row0 = qblk * (2 * NQ * BM) + r * (NQ * BM) + s * BM;
    if (row0 >= p.Lq) return 0;
    int n = nblk_all;
    if (p.causal) {
      const int last_col = row0 + (BM - 1) + (p.Lkv - p.Lq);
      const int nc = last_col < 0 ? 0 : last_col / BN + 1;
      n = nc < n ? nc : n;
    }
    return n;
  };
  int n_pair[NQ];
  int nmax = 0;
#pragma unroll
  for (int s = 0; s < NQ; ++s) {
    const int a = need(0, s), b = need(1, s);
    n_pair[s] = a > b ? a : b;
    nmax = n_pair[s] > nmax ? n_pair[s] : nmax;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < NQ; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&o_done[i], 1);
      mbar_init(&p_full[i], 256);
      mbar_init(&q_ready[i], 2);
    }
    for (int i = 0; i < NSTAGE; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&kv_ready[i], 2);
    }
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc2(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish2();
  }
  if (warp == kTmaWarp && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the barriers of both CTAs exist before anyone arrives on the peer's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const uint32_t l_p_full = mapa_shared(smem_u32(p_full), 0);
  const uint32_t l_q_ready = mapa_shared(smem_u32(q_ready), 0);
  const uint32_t l_kv_ready = mapa_shared(smem_u32(kv_ready), 0);

  if (warp >= kMmaWarp) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer (own tiles and halves)
    if (lane == 0) {
      bool ok = true;
      auto load_q = [&](int s) {
        if (n_pair[s] == 0) return;
        mbar_expect_tx(&q_full[s], Cfg::Q_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < DQK / 64; ++c)
          tma_load_3d(sQ + s * Cfg::Q_TILE_BYTES + c * (BM * 128), &tmQ, &q_full[s], c * 64, m_base + s * BM, bh);
      };
      load_q(0);
      // ring items: 2j = K block j (this CTA: keys [64 rank, 64 rank + 64)), 2j+1 = V block j (columns [64 rank, +64))
      const int nitems = 2 * nmax;
      int t_issued = 0;
      for (int t = 0; t < nitems && ok; ++t) {
        const int slot = t % NSTAGE;
        const int use = t / NSTAGE;
        if (use > 0) ok = mbar_wait(&kv_empty[slot], (use - 1) & 1, ab, kTagKvEmpty);
        if (!ok) break;
        uint8_t* dst = sKV + slot * Cfg::KV_SLOT_BYTES;
        const int j = t >> 1;
        if ((t & 1) == 0) {
          mbar_expect_tx(&kv_full[slot], Cfg::K_HALF_BYTES);
#pragma unroll
          for (int c = 0; c < DQK / 64; ++c)
            tma_load_3d(dst + c * ((BN / 2) * 128), &tmK, &kv_full[slot], c * 64, j * BN + static_cast<int>(rank) * (BN / 2), bh);
        } else {
          mbar_expect_tx(&kv_full[slot], Cfg::V_HALF_BYTES);
          tma_load_3d(dst, &tmV, &kv_full[slot], dv_off + static_cast<int>(rank) * (DV / 2), j * BN, bh);
        }
        t_issued = t + 1;
        if (t == 0) load_q(1);
      }
      if (!ok) {
        // abort path: let the copies already issued land before this CTA's shared memory is released
        for (int s = 0; s < NQ; ++s)
          if (n_pair[s] > 0 && (s == 0 || t_issued > 0)) mbar_wait_drain(&q_full[s], 0, 2000000ull);
        for (int slot = 0; slot < NSTAGE; ++slot)
          if (t_issued > slot) mbar_wait_drain(&kv_full[slot], ((t_issued - 1 - slot) / NSTAGE) & 1, 2000000ull);
      }
    }
  } else if (warp == kScoutWarp) {
    // ------------------------------------------------------------------ scout: own arrivals -> leader's barriers
    // Same order as the producer issues: Q tile 0, ring item 0, Q tile 1, ring items 1, 2, ...
    bool ok = true;
    auto relay_q = [&](int s) {
      if (n_pair[s] == 0 || !ok) return;
      ok = mbar_wait_warp(&q_full[s], 0, ab, kTagQ);
      if (ok && elect_one()) mbar_arrive_cluster(l_q_ready + s * 8);
      __syncwarp();
    };
    relay_q(0);
    const int nitems = 2 * nmax;
    for (int t = 0; t < nitems && ok; ++t) {
      const int slot = t % NSTAGE;
      ok = mbar_wait_warp(&kv_full[slot], (t / NSTAGE) & 1, ab, kTagKvFull);
      if (ok && elect_one()) mbar_arrive_cluster(l_kv_ready + slot * 8);
      __syncwarp();
      if (t == 0) relay_q(1);
    }
  } else if (warp == kMmaWarp && rank == 0) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA)
    constexpr uint32_t idesc_qk = umma_idesc(2 * BM, BN, BF16, false, false);
    constexpr uint32_t idesc_pv = umma_idesc(2 * BM, DV, BF16, false, true);
    bool ok = true;
    uint32_t ready_waited = 0;  // ring items whose kv_ready has been waited for
    auto wait_item = [&](int t) -> bool {
      while (ok && static_cast<int>(ready_waited) <= t) {
        ok = mbar_wait_warp(&kv_ready[ready_waited % NSTAGE], (ready_waited / NSTAGE) & 1, ab, kTagKvFull);
        ++ready_waited;
      }
      return ok;
    };
    const uint32_t q_addr = smem_u32(sQ);
    const uint32_t kv_addr = smem_u32(sKV);
    auto issue_s = [&](int s, int j, bool release) {
      const int slot = (2 * j) % NSTAGE;
      const uint32_t qa = q_addr + s * Cfg::Q_TILE_BYTES;
      const uint32_t ka = kv_addr + slot * Cfg::KV_SLOT_BYTES;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < DQK / 16; ++ks)
          umma_ss2(tmem_base + s * 128, umma_smem_desc(qa + (ks >> 2) * (BM * 128) + (ks & 3) * 32, 16, 1024),
                   umma_smem_desc(ka + (ks >> 2) * ((BN / 2) * 128) + (ks & 3) * 32, 16, 1024), idesc_qk, ks > 0 ? 1u : 0u);
        tc_commit2_both(&s_full[s]);
        if (release) tc_commit2_both(&kv_empty[slot]);
      }
      __syncwarp();
    };
    auto issue_pv = [&](int s, int j, bool release) {
      const int slot = (2 * j + 1) % NSTAGE;
      const uint32_t va = kv_addr + slot * Cfg::KV_SLOT_BYTES;
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < BN / 16; ++ks)
          umma_ts2(tmem_base + NQ * 128 + s * DV, tmem_base + s * 128 + ks * 8,
                   umma_smem_desc(va + ks * 2048, BN * 128, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
        tc_commit2_both(&o_done[s]);
        if (release) tc_commit2_both(&kv_empty[slot]);
      }
      __syncwarp();
    };
    int last_user = -1;
#pragma unroll
    for (int s = 0; s < NQ; ++s)
      if (n_pair[s] > 0) last_user = s;
    if (nmax > 0) {
#pragma unroll
      for (int s = 0; s < NQ; ++s) {
        if (n_pair[s] > 0 && ok) {
          ok = mbar_wait_warp(&q_ready[s], 0, ab, kTagQ);
          if (ok && wait_item(0)) {
            tc_fence_after();
            issue_s(s, 0, s == last_user);
          }
        }
      }
    }
    for (int j = 0; j < nmax && ok; ++j) {
      int last_v = -1, last_k = -1;
#pragma unroll
      for (int s = 0; s < NQ; ++s) {
        if (n_pair[s] > j) last_v = s;
        if (n_pair[s] > j + 1) last_k = s;
      }
#pragma unroll
      for (int s = 0; s < NQ; ++s) {
        if (n_pair[s] > j && ok) {
          if (!wait_item(2 * j + 1)) break;
          ok = mbar_wait_warp(&p_full[s], j & 1, ab, kTagPFull);
          if (!ok) break;
          tc_fence_after();
          issue_pv(s, j, s == last_v);
        }
        if (n_pair[s] > j + 1 && ok) {
          if (!wait_item(2 * j + 2)) break;
          tc_fence_after();
          issue_s(s, j + 1, s == last_k);
        }
      }
    }
  }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int s = warp >> 2;                    // query tile of this warpgroup
    const int row_in_tile = threadIdx.x & 127;  // TMEM lane
    const int row = m_base + s * BM + row_in_tile;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    const uint32_t tS = tmem_addr(tmem_base, lane_base, s * 128);
    const uint32_t tO = tmem_addr(tmem_base, lane_base, NQ * 128 + s * DV);
    const int n_my = n_pair[s];  // blocks this tile runs through (the pair's count; surplus blocks are fully masked)
    const int causal_shift = p.Lkv - p.Lq;

    float m_ref = -INFINITY;  // reference maximum (raw score units) the exponentials are taken against
    float l_sum = 0.f;        // running sum of exp
    bool ok = true;

    for (int j = 0; j < n_my; ++j) {
      ok = mbar_wait_warp(&s_full[s], j & 1, ab, kTagSFull);
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
      const bool diag_blk = p.causal && (n0 + BN - 1 > m_base + s * BM + causal_shift);
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
      bool need = (j == 0) || ((m_blk - m_ref) * p.scale_log2 > 8.0f);
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
          ok = mbar_wait_warp(&o_done[s], (j - 1) & 1, ab, kTagODone);
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
          const uint64_t x2 = ffma2(f2_pack(sv[cc], sv[cc + 1]), sl2, nm2);
          float e0, e1;
          if (false) {
            exp2_poly2(x2, e0, e1);  // FMA-pipe exponential for EXP_EMU of every 8 pairs
          } else {
            float x0, x1;
            f2_unpack(x2, x0, x1);
            e0 = ex2_approx(x0);
            e1 = ex2_approx(x1);
          }
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
      mbar_arrive_cluster(l_p_full + s * 8);
    }

    // epilogue: O / l  ->  global, lse
    if (ok && n_my > 0) {
      ok = mbar_wait_warp(&o_done[s], (n_my - 1) & 1, ab, kTagODone);
      if (ok) {
        tc_fence_after();
        const float inv_l = l_sum > 0.f ? 1.0f / l_sum : 0.f;
        uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (static_cast<size_t>(bh) * p.Lq + row) * p.dv_total + dv_off;
#pragma unroll
        for (int c0 = 0; c0 < DV; c0 += 32) {
          uint32_t r[32];
          tmem_ld32(tO + c0, r);
          tc_wait_ld();
          if (row < p.Lq) {
#pragma unroll
            for (int i = 0; i < 32; i += 16) {
              uint32_t v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e)
                v[e] = pack2<BF16>(__uint_as_float(r[i + 2 * e]) * inv_l, __uint_as_float(r[i + 2 * e + 1]) * inv_l);
              st_global_v8(orow + c0 + i, v);
            }
          }
        }
        if (p.lse != nullptr && dv_off == 0 && row < p.Lq) {
          p.lse[static_cast<size_t>(bh) * p.Lq + row] =
              (l_sum > 0.f) ? (m_ref * p.scale + __logf(l_sum)) : -INFINITY;
        }
      }
    } else if (ok && n_my == 0 && row < p.Lq) {
      // no visible key at all for this tile (only possible with causal and Lkv < Lq): zeros
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.o) + (static_cast<size_t>(bh) * p.Lq + row) * p.dv_total + dv_off;
      for (int c = 0; c < DV; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      if (p.lse != nullptr && dv_off == 0) p.lse[static_cast<size_t>(bh) * p.Lq + row] = -INFINITY;
    }
  }


  // common tail: every role gets here, also after an aborted wait
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // no CTA leaves while the other may still arrive on its barriers or its MMAs read this CTA's memory
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
