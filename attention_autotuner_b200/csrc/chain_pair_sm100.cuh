// CTA-pair flavour of the two-GEMM chain kernel (see chain_sm100.cuh for the algorithm and the four uses):
// a cluster of two CTAs on the two SMs of one TPC works on a 256-row resident tile with tcgen05 cta_group::2.
//
//     Z[256,128]  = R[256,K1] * C_t[128,K1]^T     each CTA: its 128 rows of R, 64 of the 128 rows of C_t
//     W           = Z .* mask .* scale (./ r)      each CTA: its 128 rows, in its own tensor memory
//     ACC[256,N2] += W[256,128] * T_t[128,N2]      each CTA: its 128 rows of ACC, N2/2 columns of T_t
//
// Against the single-CTA kernel every CTA streams half of the C and T bytes per block, so the ring of the
// same size buffers twice as many blocks (with K1 = 512 the resident tile leaves 96 KB: half a block for one
// CTA, a whole block for a pair) and the L2 -> SM traffic halves; one MMA instruction drives both SMs, so the
// issuing thread is no longer a limit.
//
// Roles per CTA as in the single-CTA kernel; the MMA warps (4: GEMM1, 5: GEMM2) work in the leader CTA
// (cluster rank 0) only. Every CTA loads its own halves with plain TMA loads; its scout warp waits for them
// and arrives on the LEADER's ready barriers (two arrivals per operand group). Completions of MMAs are
// reported with one tcgen05.commit per CTA that waits for them (own barrier and the peer's, via mapa).
#pragma once

#include "chain_common.cuh"
#include "ptx_pair.cuh"

namespace ab200 {

template <int K1_, int N2_, int MODE_, bool GENERAL_, bool BF16_>
struct ChainPairConfig {
  static constexpr int K1 = K1_;      // contraction length of GEMM1 (multiple of 64, <= 512)
  static constexpr int N2 = N2_;      // accumulator columns per pair (128 or 256); each CTA streams N2/2 of T
  static constexpr int MODE = MODE_;
  static constexpr bool GENERAL = GENERAL_;
  static constexpr bool BF16 = BF16_;
  static constexpr int K1B = K1 / 64;          // boxes per half C tile (64 rows x 64 columns, 8 KB)
  static constexpr int T2B = N2 / 128;         // boxes per half T tile (128 rows x 64 columns, 16 KB)
  static constexpr int CBOX_BYTES = 64 * 128;
  static constexpr int TBOX_BYTES = 128 * 128;
  static constexpr int ITEM_BYTES = 32768;     // a ring item: up to 4 C boxes (256 columns of K1) or the half T tile
  static constexpr int CI = (K1B + 3) / 4;     // ring items per half C tile
  static constexpr int TI = 1;
  static constexpr int R_BYTES = 128 * K1 * 2;
  static constexpr int AUX_BYTES = 2048;
  static constexpr int NSLOT_FIT = (232448 - 1024 - AUX_BYTES - R_BYTES) / ITEM_BYTES;
  static constexpr int NSLOT = NSLOT_FIT > 6 ? 6 : NSLOT_FIT;
  static constexpr int SMEM_BYTES = 1024 + R_BYTES + NSLOT * ITEM_BYTES + AUX_BYTES;
  static constexpr int NTHREADS = 384;
  static constexpr int TMEM_COLS = 512;  // 2 x 128 (Z) + N2
  static_assert(K1 % 64 == 0 && K1 >= 64 && K1 <= 512, "K1");
  static_assert(N2 == 128 || N2 == 256, "N2");
  static_assert(NSLOT >= 3, "ring too small");
  static_assert(2 * NSLOT + 24 <= 96, "barrier area");
};

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::NTHREADS, 1)
chain_pair_sm100_kernel(const __grid_constant__ CUtensorMap tmR, const __grid_constant__ CUtensorMap tmC,
                        const __grid_constant__ CUtensorMap tmT, const ChainParams p) {
  constexpr int K1B = Cfg::K1B, T2B = Cfg::T2B, N2 = Cfg::N2, NSLOT = Cfg::NSLOT, MODE = Cfg::MODE;
  constexpr int CI = Cfg::CI, TI = Cfg::TI, ITEM = Cfg::ITEM_BYTES;
  constexpr bool GENERAL = Cfg::GENERAL, BF16 = Cfg::BF16;
  constexpr int CBOX = Cfg::CBOX_BYTES, TBOX = Cfg::TBOX_BYTES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sR = smem;
  uint8_t* sRing = smem + Cfg::R_BYTES;
  float* cf = reinterpret_cast<float*>(sRing + NSLOT * ITEM);  // [2][128] column factors
  float* rs = cf + 256;                                         // [128] row sums of the finished item (forward)
  uint64_t* bars = reinterpret_cast<uint64_t*>(rs + 128);
  // "own": used in both CTAs for their own data. "leader": only the leader's copy is used; threads of both
  // CTAs arrive on it.
  uint64_t* r_full = bars;                    // own    [1] resident tile landed (transaction count)
  uint64_t* slot_full = bars + 1;             // own    [NSLOT]
  uint64_t* slot_empty = slot_full + NSLOT;   // own    [NSLOT] MMAs that read the slot completed (commit from the leader)
  uint64_t* z_full = slot_empty + NSLOT;      // own    [2] GEMM1 of a block complete
  uint64_t* w_full = z_full + 2;              // leader [2] W written by the 256 element-wise threads of the pair
  uint64_t* acc_done = w_full + 2;            // own    [1] GEMM2 of a work item complete
  uint64_t* acc_free = acc_done + 1;          // leader [1] accumulators drained by the 256 epilogue threads
  uint64_t* r_free = acc_free + 1;            // own    [1] GEMM1 of a work item complete: R may be overwritten
  uint64_t* z_free = r_free + 1;              // leader [2] GEMM2 of a block complete: its Z/W buffer may be rewritten
  uint64_t* c_ready = z_free + 2;             // leader [4] a C operand group landed in both CTAs (2 arrivals)
  uint64_t* t_ready = c_ready + 4;            // leader [4] same for a T tile
  uint64_t* r_ready = t_ready + 4;            // leader [1] resident tiles of both CTAs landed (2 arrivals)
  uint64_t* rs_free = r_ready + 1;            // own    [1] forward: row sums read by the own epilogue (128 arrivals)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(rs_free + 1);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;
  // Persistent grid of clusters: cluster c works on items c, c + n_clusters, ... of the list
  //   w = (bh * ny + chunk) * nrb + k,   256-row block = k-th heaviest  (nrb counts 256-row blocks here).
  const int rows_len = (MODE == kChainRowK) ? p.Lkv : p.Lq;
  const int cols_len = (MODE == kChainRowK) ? p.Lq : p.Lkv;
  const int ncb = (cols_len + 127) / 128;
  auto decode = [&](int w) -> ChainItem {
    ChainItem it;
    const int k = w % p.nrb;
    const int rest = w / p.nrb;
    it.n_off = (rest % p.ny) * N2;
    it.bh = rest / p.ny;
    const int rb = (p.skip_upper && MODE != kChainRowK) ? (p.nrb - 1 - k) : k;
    it.row0 = rb * 256;  // first row of the pair; this CTA owns [row0 + rank*128, +128)
    it.t_start = 0;
    it.n_iter = ncb;
    if (p.skip_upper) {
      if (MODE == kChainRowK) {
        it.t_start = 2 * rb;  // query blocks that end before this key block see none of its keys
        it.n_iter = ncb - 2 * rb;
      } else {
        it.n_iter = (2 * rb + 2 < ncb) ? 2 * rb + 2 : ncb;  // key blocks up to the one holding the last query row
      }
      if (it.n_iter < 0) it.n_iter = 0;
    }
    return it;
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
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 256);
    mbar_init(r_free, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&c_ready[i], 2);
      mbar_init(&t_ready[i], 2);
    }
    mbar_init(r_ready, 2);
    mbar_init(rs_free, 128);
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc2(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish2();
  }
  if (warp == 6 && lane == 0) {
    tma_prefetch_desc(&tmR);
    tma_prefetch_desc(&tmC);
    tma_prefetch_desc(&tmT);
  }
  tc_fence_before();
  cluster_sync();  // the barriers of both CTAs exist before anyone arrives on the peer's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const uint32_t tZ0 = tmem_base;          // Z buffers at columns [0,128) and [128,256); W overlays the first 64
  const uint32_t tACC = tmem_base + 256;   // [256, 256+N2)
  // leader's copies of the shared barriers, as shared::cluster addresses usable from both CTAs
  const uint32_t l_w_full = mapa_shared(smem_u32(w_full), 0);
  const uint32_t l_acc_free = mapa_shared(smem_u32(acc_free), 0);
  const uint32_t l_c_ready = mapa_shared(smem_u32(c_ready), 0);
  const uint32_t l_t_ready = mapa_shared(smem_u32(t_ready), 0);
  const uint32_t l_r_ready = mapa_shared(smem_u32(r_ready), 0);

  if (warp >= 4 && warp < 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
  if (warp == 6) {
    // ------------------------------------------------------------------ TMA producer (own halves)
    if (lane == 0) {
      bool ok = true;
      int bi = 0;    // ring items issued so far (all work items)
      int kacc = 0;  // non-empty work items started so far
      auto acquire = [&]() -> int {
        const int slot = bi % NSLOT;
        const int use = bi / NSLOT;
        if (use > 0) ok = mbar_wait(&slot_empty[slot], (use - 1) & 1, ab, kCtSlotEmpty);
        return slot;
      };
      for (int w = cluster_id; w < p.total_items && ok; w += n_clusters) {
        const ChainItem it = decode(w);
        if (it.n_iter == 0) continue;
        // the resident tile may be overwritten once GEMM1 of the previous item has completed
        if (kacc > 0) ok = mbar_wait(r_free, (kacc - 1) & 1, ab, kCtRFree);
        if (!ok) break;
        mbar_expect_tx(r_full, Cfg::R_BYTES);
#pragma unroll
        for (int c = 0; c < K1B; ++c) tma_load_3d(sR + c * TBOX, &tmR, r_full, c * 64, it.row0 + rank * 128, it.bh);
        ++kacc;
        if (w + n_clusters < p.total_items) {
          // the next item's resident tile usually comes from HBM: ask the L2 for it now
          const ChainItem nx = decode(w + n_clusters);
          if (nx.n_iter > 0) {
#pragma unroll
            for (int c = 0; c < K1B; ++c) tma_prefetch_3d(&tmR, c * 64, nx.row0 + rank * 128, nx.bh);
          }
        }
        // consumption order: C_0, then for t >= 1: C_t, T_{t-1}; finally T_{n-1}
        for (int t = 0; t <= it.n_iter && ok; ++t) {
          if (t < it.n_iter) {
            for (int i = 0; i < CI && ok; ++i) {
              const int slot = acquire();
              if (!ok) break;
              const int nb = (K1B - 4 * i) >= 4 ? 4 : (K1B - 4 * i);
              mbar_expect_tx(&slot_full[slot], nb * CBOX);
              for (int b = 0; b < nb; ++b)
                tma_load_3d(sRing + slot * ITEM + b * CBOX, &tmC, &slot_full[slot], (4 * i + b) * 64,
                            (it.t_start + t) * 128 + rank * 64, it.bh);
              ++bi;
            }
          }
          if (t >= 1 && ok) {
            const int slot = acquire();
            if (!ok) break;
            mbar_expect_tx(&slot_full[slot], T2B * TBOX);
            for (int b = 0; b < T2B; ++b)
              tma_load_3d(sRing + slot * ITEM + b * TBOX, &tmT, &slot_full[slot], it.n_off + rank * (N2 / 2) + b * 64,
                          (it.t_start + t - 1) * 128, it.bh);
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
  } else if (warp == 7) {
    // ------------------------------------------------------------------ scout (own halves -> leader's barriers)
    // Walks the ring in order, waits for every own item to land and arrives once per operand group on the
    // leader's ready barrier, which completes when both CTAs have arrived.
    bool ok = true;
    int bi = 0;
    int cg = 0, tg = 0, kacc = 0;
    auto post = [&](int nitems, uint32_t ready_base, int& counter) {
      for (int i0 = 0; i0 < nitems && ok; i0 += 2) {
        for (int i = i0; i < nitems && i < i0 + 2 && ok; ++i, ++bi)
          ok = mbar_wait_warp(&slot_full[bi % NSLOT], (bi / NSLOT) & 1, ab, kCtSlotFull);
        if (ok && elect_one()) mbar_arrive_cluster(ready_base + (counter & 3) * 8);
        __syncwarp();
        ++counter;
      }
    };
    for (int w = cluster_id; w < p.total_items && ok; w += n_clusters) {
      const ChainItem it = decode(w);
      const int n = it.n_iter;
      if (n == 0) continue;
      ok = mbar_wait_warp(r_full, kacc & 1, ab, kCtR);
      if (ok && elect_one()) mbar_arrive_cluster(l_r_ready);
      __syncwarp();
      ++kacc;
      for (int t = 0; t <= n && ok; ++t) {
        if (t < n) post(CI, l_c_ready, cg);
        if (t >= 1) post(TI, l_t_ready, tg);
      }
    }
  }
  else if ((warp == 4 || warp == 5) && rank == 0) {
    // ------------------------------------------------------------------ MMA issuers (leader CTA only)
    // Warp 4 issues GEMM1 (Z), warp 5 GEMM2 (ACC); converged warps, one elected lane issues. Ring items are
    // consumed in a fixed order:  C_0 at b0;  C_t at b0 + CI + (t-1)(CI+TI);  T_t right after C_{t+1}, except
    // the last T_{n-1}, which follows T_{n-2} directly. Both CTAs keep identical rings, so one slot index
    // addresses the operand halves of both.
    constexpr uint32_t idesc_z = umma_idesc(256, 128, BF16, false, false);
    constexpr uint32_t idesc_acc = umma_idesc(256, N2, BF16, false, true);
    bool ok = true;
    int b0 = 0;    // ring items of earlier work items
    int g0 = 0;    // 128-wide blocks of earlier work items (selects Z buffer and ready barrier)
    int kacc = 0;  // non-empty work items finished so far
    int cg = 0, tg = 0;  // operand groups consumed so far (as the scouts count them)
    const uint32_t r_addr = smem_u32(sR);
    const uint32_t ring_addr = smem_u32(sRing);
    for (int w = cluster_id; w < p.total_items && ok; w += n_clusters) {
      const ChainItem it = decode(w);
      const int n = it.n_iter;
      if (n == 0) continue;
      if (warp == 4) {
        ok = mbar_wait_warp(r_ready, kacc & 1, ab, kCtR);
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
                  const int nb = (K1B - 4 * i) >= 4 ? 4 : (K1B - 4 * i);
#pragma unroll
                  for (int b = 0; b < 4; ++b) {
                    if (b < nb) {
#pragma unroll
                      for (int ks = 0; ks < 4; ++ks)
                        umma_ss2(tz, umma_smem_desc(r_addr + (4 * i + b) * TBOX + ks * 32, 16, 1024),
                                 umma_smem_desc(a + b * CBOX + ks * 32, 16, 1024), idesc_z,
                                 (i > 0 || b > 0 || ks > 0) ? 1u : 0u);
                    }
                  }
                  tc_commit2_both(&slot_empty[slot]);
                }
              }
              if (i0 + 2 >= CI) {
                tc_commit2_both(&z_full[g & 1]);
                if (t + 1 == n) tc_commit2_both(r_free);
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
            // the first GEMM2 overwrites the accumulators: both epilogues of the previous item must have read them
            ok = mbar_wait_warp(acc_free, (kacc - 1) & 1, ab, kCtAccFree);
            if (!ok) break;
          }
          ok = mbar_wait_warp(&w_full[g & 1], (g >> 1) & 1, ab, kCtWFull);
          if (!ok) break;
          if (lane == 0) AB200_CTR(1, g, 2);
          const uint32_t tw = tZ0 + (g & 1) * 128;
          const int base = b0 + CI + t * (CI + TI) + (t + 1 < n ? CI : 0);
          ok = mbar_wait_warp(&t_ready[tg & 3], (tg >> 2) & 1, ab, kCtSlotFull);
          ++tg;
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            const int slot = base % NSLOT;
            const uint32_t a = ring_addr + slot * ITEM;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_ts2(tACC, tw + ks * 8, umma_smem_desc(a + ks * 2048, TBOX, 1024), idesc_acc, (t > 0 || ks > 0) ? 1u : 0u);
            tc_commit2_both(&slot_empty[slot]);
            tc_commit2(smem_u32(&z_free[g & 1]));
            if (t + 1 == n) tc_commit2_both(acc_done);
          }
          __syncwarp();
          if (lane == 0) AB200_CTR(1, g, 3);
        }
      }
      b0 += n * (CI + TI);
      g0 += n;
      ++kacc;
    }
  }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ element-wise warpgroup (own 128 rows)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int tid = threadIdx.x;  // 0..127 = TMEM lane = row of the CTA's tile
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32);
    constexpr bool decay_mode = !GENERAL;
    bool ok = true;
    int g0 = 0;     // blocks processed before the current work item
    int kacc = 0;   // non-empty work items finished so far
    int kitem = 0;  // work items seen so far (selects the per-item column-factor table)

    for (int w = cluster_id; w < p.total_items && ok; w += n_clusters, ++kitem) {
      const ChainItem it = decode(w);
      const int bh = it.bh, row0 = it.row0 + static_cast<int>(rank) * 128, n_off = it.n_off, t_start = it.t_start;
      const int n_iter = it.n_iter;
      const int grow = row0 + tid;  // global row index on the row side
      const int h = bh % p.H;
      float lg = 0.f;  // log2(gamma)
      if (decay_mode) lg = log2f(p.decay[h]);
      float rowf_base = p.scale;
      if (decay_mode) rowf_base *= exp2f((MODE == kChainRowK ? -tid : tid) * lg);
      if (MODE == kChainRowQ) rowf_base *= (grow < p.Lq) ? 1.0f / p.r_in[static_cast<size_t>(bh) * p.Lq + grow] : 0.f;
      const float* cf_item = cf + (kitem & 1) * 128;
      if (MODE != kChainRowK && decay_mode) {
        cf[(kitem & 1) * 128 + tid] = exp2f(-tid * lg);
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      float rsum = 0.f;
      if (n_iter == 0) {
        // no block contributes to this tile: zeros (and r = 1 in the forward)
        if (grow < rows_len) {
          uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * rows_len + grow) * p.ld_out + n_off;
          for (int c = 0; c < N2; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
          if (MODE == kChainFwd && n_off == 0) p.r_out[static_cast<size_t>(bh) * p.Lq + grow] = 1.0f;
        }
        continue;
      }

      for (int t = 0; t < n_iter; ++t) {
        const int g = g0 + t;  // running block index: Z buffer g & 1
        const int col0 = (t_start + t) * 128;
        const float* cft = cf_item;
        if (MODE == kChainRowK) {
          // column factor: 1/r of the block's queries (times gamma^c under decay)
          const int qi = col0 + tid;
          float f = (qi < p.Lq) ? 1.0f / p.r_in[static_cast<size_t>(bh) * p.Lq + qi] : 0.f;
          if (decay_mode) f *= exp2f(tid * lg);
          cf[(g & 1) * 128 + tid] = f;
          asm volatile("bar.sync 1, 128;" ::: "memory");
          cft = cf + (g & 1) * 128;
        }
        float rowf = rowf_base;
        if (decay_mode) rowf *= exp2f((MODE == kChainRowK ? (col0 - row0) : (row0 - col0)) * lg);
        //   Fwd/RowQ: column c valid iff col0 + c <= grow ;  RowK: valid iff col0 + c >= grow
        const bool straddle = decay_mode && (MODE == kChainRowK ? (col0 < row0 + 127) : (col0 + 127 > row0));
        const int dlim = grow - col0;

        if (tid == 0) AB200_CTR(0, g, 0);
        ok = mbar_wait_warp(&z_full[g & 1], (g >> 1) & 1, ab, kCtZFull);
        if (!ok) break;
        if (tid == 0) AB200_CTR(0, g, 1);
        tc_fence_after();
        const uint32_t tz = tmem_addr(tZ0 + (g & 1) * 128, lane_base, 0);
        chain_ew_block<MODE, GENERAL, BF16>(p, tz, cft, rowf, straddle, dlim, grow, col0, h, rsum);
        if (MODE == kChainFwd && t + 1 == n_iter) {
          // hand the row sums to the own epilogue warpgroup (single buffer: it must have read the previous ones)
          if (kacc > 0) {
            ok = mbar_wait_warp(rs_free, (kacc - 1) & 1, ab, kCtAccFree);
            if (!ok) break;
          }
          rs[tid] = rsum;
        }
        if (tid == 0) AB200_CTR(0, g, 2);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive_cluster(l_w_full + (g & 1) * 8);
        if (tid == 0) AB200_CTR(0, g, 3);
      }
      if (!ok) break;
      g0 += n_iter;
      ++kacc;
    }
  } else {
    // ------------------------------------------------------------------ epilogue warpgroup (own 128 rows)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 112;");
    const int tid = threadIdx.x - 256;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    bool ok = true;
    int kacc = 0;
    for (int w = cluster_id; w < p.total_items && ok; w += n_clusters) {
      const ChainItem it = decode(w);
      if (it.n_iter == 0) continue;  // the element-wise warpgroup writes the zeros of an empty tile
      const int grow = it.row0 + static_cast<int>(rank) * 128 + tid;
      uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(it.bh) * rows_len + grow) * p.ld_out + it.n_off;
      ok = mbar_wait_warp(acc_done, kacc & 1, ab, kCtAccDone);
      if (!ok) break;
      tc_fence_after();
      float osc = 1.0f;
      if (MODE == kChainFwd) {
        const float r = fmaxf(rs[tid], 1.0f);
        mbar_arrive(rs_free);
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
          mbar_arrive_cluster(l_acc_free);
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
  tc_fence_before();
  cluster_sync();  // no CTA leaves while the other may still arrive on its barriers or its MMAs read this CTA's memory
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
