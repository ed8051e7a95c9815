// flash-attention forward for sm_100a:  O = softmax(Q K^T * scale [+ causal mask]) V,  LSE optional.
//
// Replaces the reference kernels flashattn_fwd_regfuse (csrc/kernels/attention/regfuse/regfuse.h:48-455)
// and flashattn_fwd_smemfuse (csrc/kernels/attention/smemfuse/smemfuse.h:61-614). On Blackwell the
// accumulators live in tensor memory, which replaces both of the reference's fusion styles.
//
// One CTA owns NQ (1 or 2) query tiles of 128 rows of one (batch, head) slice and walks the KV sequence
// in blocks of 128 keys.
//   warps 0..4*NQ-1 : one softmax warpgroup per query tile; thread t owns row t of its tile, so row
//                     statistics need no shuffles. Reads S from TMEM, writes P (16-bit) back into the
//                     same TMEM columns, rescales O in TMEM on the rare steps where the running maximum
//                     moved by more than 2^8 ("lazy" rescale), runs the epilogue.
//   warp 4*NQ       : lane 0 issues every tcgen05.mma: S = Q K^T (both operands from shared memory,
//                     K-major) and O += P V (P from TMEM, V from shared memory, MN-major).
//   warp 4*NQ+1     : lane 0 is the TMA producer: Q tiles once, then K/V tiles through a ring.
// With NQ = 2 the two query tiles ping-pong: while warpgroup 0 does the softmax of its tile, the tensor
// pipe runs the two GEMMs of tile 1, and vice versa.
//
// TMEM columns (fp32): S tile s at [128*s, 128*s+128), P tile s overlays the first 64 columns of S
// tile s (two 16-bit values per column), O tile s at [128*NQ + DV*s, ...).
#pragma once

#include "ptx.cuh"

namespace ab200 {

struct FaFwdParams {
  void* o;      // [BH, Lq, dv_total] storage dtype
  float* lse;   // [BH, Lq] fp32 or nullptr
  int dv_total; // full head dim of V/O; CTA z handles columns [z*DV, z*DV+DV)
  int Lq;
  int Lkv;
  int causal;          // 0/1; bottom-right aligned when Lq != Lkv (key j visible to row i iff j <= i + Lkv - Lq)
  float scale;         // softmax scale
  float scale_log2;    // scale * log2(e)
};

template <int DQK_, int DV_, int NQ_, int NSTAGE_, bool BF16_, int EXP_EMU_ = 0, int SPLIT_ = 1, int NMMA_ = 1, int EXP_H2_ = 0>
struct FaFwdConfig {
  // of every 4 groups of 8 scores, how many take the packed half-precision exponential (ex2.approx.f16x2: two
  // results per MUFU operation, already in P's storage type). fp16 only; 0 = every exponential in fp32. MUFU is
  // as scarce as the tensor pipe at head dimension 128 (one ex2 per 256 tensor FLOP, 16 per clock and SM), so this
  // halves the longest phase of the softmax. The argument of the exponential is rounded to fp16 first, whose
  // precision falls with |x|: configurations that use it keep the lazy-rescale threshold at 2^4 instead of 2^8, so
  // that the entries that dominate a row have |x| < 4 (relative error below 6.8e-4, against 4.9e-4 for rounding P
  // itself to fp16). Row sums of these groups are added in fp16 over four pairs (values below 2^5) and
  // accumulated in fp32.
  static constexpr int EXP_H2 = EXP_H2_;
  static_assert(EXP_H2_ >= 0 && EXP_H2_ <= 4, "EXP_H2 counts groups out of 4");
  static_assert(EXP_H2_ == 0 || (!BF16_ && SPLIT_ == 1 && EXP_EMU_ == 0), "EXP_H2 needs fp16, one softmax warpgroup per tile, no FMA-pipe emulation");
  // log2 of the growth of the running maximum that triggers a rescale of O
  static constexpr float RESCALE_LOG2 = EXP_H2_ > 0 ? 4.0f : 8.0f;
  // MMA-issuing warps: 1, or 2 taking strict turns, one per query tile (see fa_fwd_mma_pair.cuh)
  static constexpr int NMMA = NMMA_;
  static_assert(NMMA_ == 1 || (NMMA_ == 2 && NQ_ == 2), "NMMA");
  // softmax warpgroups per query tile: 1 (a thread owns a whole 128-column score row) or 2 (two threads share a
  // row, 64 columns each, and exchange the row maximum through shared memory): halves the serial softmax time of
  // a tile, which is what the tensor pipe waits for
  static constexpr int SPLIT = SPLIT_;
  static_assert(SPLIT_ == 1 || (SPLIT_ == 2 && NQ_ == 2 && DV_ % 64 == 0), "SPLIT");
  // of every 8 pairs of scores, how many take the FMA-pipe exponential instead of MUFU ex2 (0..8). Measured
  // on B200 at d = 128: every non-zero setting is slower (the softmax warps are issue/latency bound, not
  // MUFU bound), so the default is 0; kept as a tuning knob.
  static constexpr int EXP_EMU = EXP_EMU_;
  static constexpr int DQK = DQK_;        // head dim of Q/K, multiple of 64
  static constexpr int DV = DV_;          // head dim of V/O, multiple of 64
  static constexpr int NQ = NQ_;          // query tiles per CTA
  static constexpr int NSTAGE = NSTAGE_;  // K/V ring depth (entries of one K or one V tile)
  static constexpr bool BF16 = BF16_;
  static constexpr int BM = 128;          // rows per query tile
  static constexpr int BN = 128;          // keys per KV block
  static constexpr int NTHREADS = 128 * NQ * SPLIT + 128;  // softmax warpgroups + one auxiliary warpgroup (MMA, TMA, 2 idle warps)
  static constexpr int Q_TILE_BYTES = BM * DQK * 2;
  static constexpr int K_TILE_BYTES = BN * DQK * 2;
  static constexpr int V_TILE_BYTES = BN * DV * 2;
  static constexpr int KV_SLOT_BYTES = K_TILE_BYTES > V_TILE_BYTES ? K_TILE_BYTES : V_TILE_BYTES;
  static constexpr int TMEM_COLS_USED = NQ * (128 + DV);
  static constexpr int TMEM_COLS = TMEM_COLS_USED <= 32 ? 32 : TMEM_COLS_USED <= 64 ? 64 : TMEM_COLS_USED <= 128 ? 128 : TMEM_COLS_USED <= 256 ? 256 : 512;
  static constexpr int SMEM_TILES = NQ * Q_TILE_BYTES + NSTAGE * KV_SLOT_BYTES;
  static constexpr int XCHG_BYTES = SPLIT == 2 ? NQ * 3 * 2 * 128 * 4 : 0;  // row max (double buffered) and row sum exchange
  static constexpr int SMEM_BYTES = SMEM_TILES + 1024 /*alignment slack*/ + 256 /*barriers*/ + XCHG_BYTES;
  static_assert(DQK % 64 == 0 && DV % 64 == 0, "head dims must be multiples of 64");
  static_assert(TMEM_COLS_USED <= 512, "TMEM overflow: NQ*(128+DV) must be <= 512 columns");
  static_assert(DV <= 256, "one PV MMA covers at most N=256");
  static_assert(SMEM_BYTES <= 232448, "shared memory overflow");
};

// Optional event trace (compile with -DAB200_TRACE): CTA (0,0,0) records clock64() at the hand-off points of
// softmax warp 0 of each tile and of the MMA thread, for the first kTraceIters KV blocks.
#ifdef AB200_TRACE
constexpr int kTraceIters = 16;
__device__ long long g_trace[5][kTraceIters][8];
#define AB200_TR(who, j, ev)                                                                       \
  do {                                                                                             \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < kTraceIters) g_trace[who][j][ev] = clock64(); \
  } while (0)
#else
#define AB200_TR(who, j, ev) do {} while (0)
#endif

// Barrier tags reported with a timeout status.
enum FaTag : int { kTagQ = 1, kTagKvFull = 2, kTagKvEmpty = 3, kTagSFull = 4, kTagPFull = 5, kTagODone = 6, kTagTurn = 7 };

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
fa_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const FaFwdParams p) {
  constexpr int DQK = Cfg::DQK, DV = Cfg::DV, NQ = Cfg::NQ, NSTAGE = Cfg::NSTAGE;
  constexpr bool BF16 = Cfg::BF16;
  constexpr int BM = Cfg::BM, BN = Cfg::BN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + NQ * Cfg::Q_TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::SMEM_TILES);
  uint64_t* q_full = bars;                   // [NQ]
  uint64_t* kv_full = q_full + NQ;           // [NSTAGE]
  uint64_t* kv_empty = kv_full + NSTAGE;     // [NSTAGE]
  uint64_t* s_full = kv_empty + NSTAGE;      // [NQ]
  uint64_t* p_full = s_full + NQ;            // [NQ]
  uint64_t* o_done = p_full + NQ;            // [NQ]
  uint64_t* turn = o_done + NQ;              // [2] issue turns of the two MMA warps (NMMA == 2)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(turn + 2);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);
  float* xchg = reinterpret_cast<float*>(smem + Cfg::SMEM_TILES + 256);  // [NQ][3][2][128], SPLIT == 2 only

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
  const int lane = threadIdx.x & 31;
  constexpr int SPLIT = Cfg::SPLIT;
  constexpr int kMmaWarp = 4 * NQ * SPLIT;
  constexpr int NMMA = Cfg::NMMA;
  constexpr int kTmaWarp = 4 * NQ * SPLIT + NMMA;

  // Heaviest (latest) query blocks first under a causal mask.
  const int qblk = p.causal ? (gridDim.x - 1 - blockIdx.x) : blockIdx.x;
  // grid: x = query block, y = V-column chunk, z = (batch, head)
  const int bh = blockIdx.z;
  const int dv_off = blockIdx.y * DV;
  const int m_base = qblk * (BM * NQ);

  // KV blocks needed per query tile.
  const int nblk_all = (p.Lkv + BN - 1) / BN;
  int nblk[NQ];
  int nmax = 0;
#pragma unroll
  for (int s = 0; s < NQ; ++s) {
    int n = nblk_all;
    if (p.causal) {
      const int last_col = m_base + s * BM + (BM - 1) + (p.Lkv - p.Lq);
      int nc = last_col < 0 ? 0 : last_col / BN + 1;
      n = nc < n ? nc : n;
    }
    if (m_base + s * BM >= p.Lq) n = 0;  // tile entirely past the end of Q
    nblk[s] = n;
    nmax = n > nmax ? n : nmax;
  }

  if (threadIdx.x == 0) {
    for (int i = 0; i < NQ; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128 * SPLIT);
      mbar_init(&o_done[i], 1);
    }
    for (int i = 0; i < NSTAGE; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], NMMA);
    }
    mbar_init(&turn[0], 1);
    mbar_init(&turn[1], 1);
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

  // With three warpgroups the launch-time register split (168/thread) starves the softmax threads, which
  // hold a full 128-column score row; each role branch moves registers accordingly (setmaxnreg).
  if (warp >= kMmaWarp) {
    // (setmaxnreg.inc waits, with no limit, until the registers it asks for have been released: 256 x 208 for the
    // softmax threads + 128 x 72 here must not exceed the 384 x 168 the CTA was given)
    static_assert(256 * 208 + 128 * 72 <= 384 * 168, "register split of the warpgroups");
    if constexpr (NQ == 2 && SPLIT == 1) asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
  if (warp == kTmaWarp) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      auto load_q = [&](int s) {
        if (nblk[s] == 0) return;
        mbar_expect_tx(&q_full[s], Cfg::Q_TILE_BYTES);
#pragma unroll
        for (int c = 0; c < DQK / 64; ++c)
          tma_load_3d(sQ + s * Cfg::Q_TILE_BYTES + c * (BM * 128), &tmQ, &q_full[s], c * 64, m_base + s * BM, bh);
      };
      load_q(0);
      // ring items: 2j = K block j, 2j+1 = V block j
      const int nitems = 2 * nmax;
      int t_issued = 0;
      for (int t = 0; t < nitems && ok; ++t) {
        const int slot = t % NSTAGE;
        const int use = t / NSTAGE;
        AB200_TR(3, t >> 1, (t & 1) * 4 + 0);
        if (use > 0) ok = mbar_wait(&kv_empty[slot], (use - 1) & 1, ab, kTagKvEmpty);
        if (!ok) break;
        AB200_TR(3, t >> 1, (t & 1) * 4 + 1);
        uint8_t* dst = sKV + slot * Cfg::KV_SLOT_BYTES;
        const int j = t >> 1;
        if ((t & 1) == 0) {
          mbar_expect_tx(&kv_full[slot], Cfg::K_TILE_BYTES);
#pragma unroll
          for (int c = 0; c < DQK / 64; ++c) tma_load_3d(dst + c * (BN * 128), &tmK, &kv_full[slot], c * 64, j * BN, bh);
        } else {
          mbar_expect_tx(&kv_full[slot], Cfg::V_TILE_BYTES);
#pragma unroll
          for (int c = 0; c < DV / 64; ++c) tma_load_3d(dst + c * (BN * 128), &tmV, &kv_full[slot], dv_off + c * 64, j * BN, bh);
        }
        t_issued = t + 1;
        if (t == 0) {
#pragma unroll
          for (int s = 1; s < NQ; ++s) load_q(s);
        }
      }
      if (!ok) {
        // abort path: let the copies already issued land before this CTA's shared memory is released
        for (int s = 0; s < NQ; ++s)
          if (nblk[s] > 0 && (s == 0 || t_issued > 0)) mbar_wait_drain(&q_full[s], 0, 2000000ull);
        for (int slot = 0; slot < NSTAGE; ++slot) {
          if (t_issued > slot) mbar_wait_drain(&kv_full[slot], ((t_issued - 1 - slot) / NSTAGE) & 1, 2000000ull);
        }
      }
    }
  } else if (NMMA == 2 && warp < kMmaWarp + 2) {
    // ------------------------------------------------------------------ MMA issuers, one per query tile
    if constexpr (NMMA == 2) {
#include "fa_fwd_mma_pair.cuh"
    }
  } else if (NMMA == 1 && warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs this role converged (waits included); one elected lane issues each batch of
    // tcgen05.mma + commits, so that addresses and descriptors stay warp-uniform.
    {
      constexpr uint32_t idesc_qk = umma_idesc(BM, BN, BF16, false, false);
      constexpr uint32_t idesc_pv = umma_idesc(BM, DV, BF16, false, true);
      bool ok = true;
      uint32_t full_waited = 0;  // number of ring items whose kv_full has been waited for
      auto wait_item = [&](int t) -> bool {
        // ring items are consumed in order; wait for every item up to t exactly once
        while (ok && static_cast<int>(full_waited) <= t) {
          const int slot = full_waited % NSTAGE;
          const int use = full_waited / NSTAGE;
          if (lane == 0) AB200_TR(4, full_waited >> 1, (full_waited & 1) * 4 + 0);
          ok = mbar_wait_warp(&kv_full[slot], use & 1, ab, kTagKvFull);
          if (lane == 0) AB200_TR(4, full_waited >> 1, (full_waited & 1) * 4 + 1);
          ++full_waited;
        }
        return ok;
      };
      const uint32_t q_addr = smem_u32(sQ);
      const uint32_t kv_addr = smem_u32(sKV);
      // S_s = Q_s K_j^T, then optionally release the K slot
      auto issue_s = [&](int s, int j, bool release) {
        const int slot = (2 * j) % NSTAGE;
        const uint32_t qa = q_addr + s * Cfg::Q_TILE_BYTES;
        const uint32_t ka = kv_addr + slot * Cfg::KV_SLOT_BYTES;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < DQK / 16; ++ks) {
            const uint32_t off = (ks >> 2) * (BM * 128) + (ks & 3) * 32;
            umma_ss(tmem_base + s * 128, umma_smem_desc(qa + off, 16, 1024), umma_smem_desc(ka + off, 16, 1024),
                    idesc_qk, ks > 0 ? 1u : 0u);
          }
          tc_commit(&s_full[s]);
          if (release) tc_commit(&kv_empty[slot]);
        }
        __syncwarp();
      };
      // O_s += P_s V_j, then optionally release the V slot
      auto issue_pv = [&](int s, int j, bool release) {
        const int slot = (2 * j + 1) % NSTAGE;
        const uint32_t va = kv_addr + slot * Cfg::KV_SLOT_BYTES;
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < BN / 16; ++ks) {
            // P sits in the first 64 columns of the S region; with two softmax warpgroups per tile each half keeps
            // its 32 P columns inside its own score columns: [0,32) and [64,96)
            const uint32_t pcol = (SPLIT == 2 && ks >= 4) ? 64 + (ks - 4) * 8 : ks * 8;
            umma_ts(tmem_base + NQ * 128 + s * DV, tmem_base + s * 128 + pcol,
                    umma_smem_desc(va + ks * 2048, BN * 128, 1024), idesc_pv, (j > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(&o_done[s]);
          if (release) tc_commit(&kv_empty[slot]);
        }
        __syncwarp();
      };
      int last_user = -1;
      // prologue: S_s(0)
#pragma unroll
      for (int s = 0; s < NQ; ++s)
        if (nblk[s] > 0) last_user = s;
      if (nmax > 0) {
#pragma unroll
        for (int s = 0; s < NQ; ++s) {
          if (nblk[s] > 0 && ok) {
            ok = mbar_wait_warp(&q_full[s], 0, ab, kTagQ);
            if (ok && wait_item(0)) {
              tc_fence_after();
              issue_s(s, 0, s == last_user);
            }
          }
        }
      }
      for (int j = 0; j < nmax && ok; ++j) {
        // users of V_j are the tiles with nblk > j; users of K_{j+1} those with nblk > j+1
        int last_v = -1, last_k = -1;
#pragma unroll
        for (int s = 0; s < NQ; ++s) {
          if (nblk[s] > j) last_v = s;
          if (nblk[s] > j + 1) last_k = s;
        }
#pragma unroll
        for (int s = 0; s < NQ; ++s) {
          if (nblk[s] > j && ok) {
            if (!wait_item(2 * j + 1)) break;
            if (lane == 0) AB200_TR(2, j, s * 4 + 0);
            ok = mbar_wait_warp(&p_full[s], j & 1, ab, kTagPFull);
            if (!ok) break;
            if (lane == 0) AB200_TR(2, j, s * 4 + 1);
            tc_fence_after();
            issue_pv(s, j, s == last_v);
            if (lane == 0) AB200_TR(2, j, s * 4 + 2);
          }
          if (nblk[s] > j + 1 && ok) {
            if (!wait_item(2 * j + 2)) break;
            tc_fence_after();
            issue_s(s, j + 1, s == last_k);
            if (lane == 0) AB200_TR(2, j, s * 4 + 3);
          }
        }
      }
    }
  }
  } else if constexpr (SPLIT == 2) {
    // ------------------------------------------------------------------ softmax warpgroups, two per query tile
#include "fa_fwd_softmax_split.cuh"
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    if constexpr (NQ == 2) asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int s = warp >> 2;                    // query tile of this warpgroup
    const int row_in_tile = threadIdx.x & 127;  // TMEM lane
    const int row = m_base + s * BM + row_in_tile;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    const uint32_t tS = tmem_addr(tmem_base, lane_base, s * 128);
    const uint32_t tO = tmem_addr(tmem_base, lane_base, NQ * 128 + s * DV);
    const int n_my = nblk[s];
    const int causal_shift = p.Lkv - p.Lq;

    float m_ref = -INFINITY;  // reference maximum (raw score units) the exponentials are taken against
    float l_sum = 0.f;        // running sum of exp
    bool ok = true;

    for (int j = 0; j < n_my; ++j) {
      if (threadIdx.x % 128 == 0) AB200_TR(s, j, 0);
      ok = mbar_wait_warp(&s_full[s], j & 1, ab, kTagSFull);
      if (!ok) break;
      if (threadIdx.x % 128 == 0) AB200_TR(s, j, 1);
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
      if (threadIdx.x % 128 == 0) AB200_TR(s, j, 2);
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
      if (threadIdx.x % 128 == 0) AB200_TR(s, j, 3);

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
      uint32_t hsum = 0;  // fp16 pair: sum of up to four packed exponentials of a group (EXP_H2)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t pk[BN / 4];
#pragma unroll
        for (int c = 0; c < BN / 2; c += 2) {
          const int cc = h * (BN / 2) + c;
          const uint64_t x2 = ffma2(f2_pack(sv[cc], sv[cc + 1]), sl2, nm2);
          if constexpr (Cfg::EXP_H2 > 0) {
            // groups of four pairs (8 scores): EXP_H2 of every 4 groups use the packed fp16 exponential
            if (((c >> 3) & 3) < Cfg::EXP_H2) {
              float x0, x1;
              f2_unpack(x2, x0, x1);
              const uint32_t ph = ex2_approx_h2(pack2<false>(x0, x1));
              pk[c >> 1] = ph;
              if (((c >> 1) & 3) == 0) hsum = ph;
              else hsum = hadd2_u32(hsum, ph);
              if (((c >> 1) & 3) == 3) acc[(c >> 3) & 3] = fadd2(acc[(c >> 3) & 3], h2_to_f2(hsum));
              continue;
            }
          }
          float e0, e1;
          if (((c >> 1) & 7) < Cfg::EXP_EMU) {
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
      if (threadIdx.x % 128 == 0) AB200_TR(s, j, 4);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&p_full[s]);
      if (threadIdx.x % 128 == 0) AB200_TR(s, j, 5);
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
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
