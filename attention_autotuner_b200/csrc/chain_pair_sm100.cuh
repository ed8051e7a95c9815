// CTA-pair flavour of the two-GEMM chain kernel (see chain_sm100.cuh for the algorithm and the four uses):
// a cluster of two CTAs on the two SMs of one TPC works on a 256-row resident tile with tcgen05 cta_group::2.
//
//     Z[256,128]  = R[256,K1] * C_t[128,K1]^T     each CTA: its 128 rows of R, 64 of the 128 rows of C_t
//     W           = Z .* mask .* scale (./ r)      each CTA: its 128 rows, in its own tensor memory
//     ACC[256,N2] += W[256,128] * T_t[128,N2]      each CTA: its 128 rows of ACC, half of the columns of T_t
//
// Against the single-CTA kernel every CTA streams half of the C and T bytes per block, so the ring of the
// same size buffers twice as many blocks (with K1 = 512 the resident tile leaves 96 KB: half a block for one
// CTA, a whole block for a pair) and the L2 -> SM traffic halves; one MMA instruction drives both SMs, so the
// issuing thread is no longer a limit.
//
// 16 warps per CTA:
//   0-3   element-wise warpgroup A: thread t owns row t, columns [0,64) of the block
//   4, 5  MMA issuers (GEMM1, GEMM2): leader CTA (cluster rank 0) only, converged warps, one elected lane
//   6     TMA producer (lane 0): this CTA's halves of the operands, ring of 16 KB items
//   7     scout: waits for this CTA's ring items and arrives on the LEADER's ready barriers (2 arrivals per group)
//   8-11  element-wise warpgroup B: row t, columns [64,128)
//   12-15 epilogue warpgroup: accumulator -> 16-bit -> shared memory -> TMA store
// Two threads per row halve the latency of the element-wise step, which sits on the critical chain
// GEMM1(t) -> W(t) -> GEMM2(t) -> GEMM1(t+2) (the block buffers in tensor memory are only two deep).
// The epilogue stages its output in the ring slots that held the last T tile of the work item (GEMM2 leaves
// them to the epilogue instead of returning them to the producer) and writes it with TMA stores: per-row
// global stores from registers (one 32-byte sector per lane) kept the accumulator busy for ~4500 cycles and
// slowed the element-wise warps of the next item through the shared load/store path.
// Completions of MMAs are reported with one tcgen05.commit per CTA that waits for them (own barrier and the
// peer's, via mapa); every CTA loads its own operand halves with plain TMA loads.
#pragma once

#include "chain_common.cuh"
#include "ptx_pair.cuh"

namespace ab200 {

template <int K1_, int N2_, int MODE_, bool GENERAL_, bool BF16_>
struct ChainPairConfig {
  static constexpr int K1 = K1_;      // contraction length of GEMM1 (multiple of 64, <= 512)
  static constexpr int N2 = N2_;      // accumulator columns per pair (128 or 256)
  static constexpr int MODE = MODE_;
  static constexpr bool GENERAL = GENERAL_;
  static constexpr bool BF16 = BF16_;
  static constexpr int K1B = K1 / 64;          // boxes per half C tile (64 rows x 64 columns, 8 KB)
  static constexpr int CBOX_BYTES = 64 * 128;
  static constexpr int TBOX_BYTES = 128 * 128;
  static constexpr int ITEM_BYTES = 16384;     // a ring item: two C boxes (128 columns of K1) or one T box (64 columns)
  static constexpr int CI = (K1B + 1) / 2;     // ring items per half C tile
  static constexpr int TI = N2 / 128;          // ring items per half T tile: item j feeds ACC columns [128j, 128j+128)
  static constexpr int R_BYTES = 128 * K1 * 2;
  static constexpr int AUX_BYTES = 2048;
  static constexpr int NSLOT_FIT = (232448 - 1024 - AUX_BYTES - R_BYTES) / ITEM_BYTES;
  static constexpr int NSLOT = NSLOT_FIT > 12 ? 12 : NSLOT_FIT;
  static constexpr int NREADY = 8;             // depth of the ready-barrier rings (groups of up to two items)
  static constexpr int SMEM_BYTES = 1024 + R_BYTES + NSLOT * ITEM_BYTES + AUX_BYTES;
  // Output staging of the epilogue: 2 * TI boxes of 16 KB. With a deep ring the boxes of a work item are staged at
  // once, in the slots of its last T tile and of the first TI items of its last C tile; with a shallow ring
  // (K1 = 512) in two rounds through the T slots only, so that the next item's first C tile is not held up.
  static constexpr bool ONE_ROUND = (CI >= TI) && (NSLOT >= 2 * (CI + TI));
  static constexpr int NTHREADS = 512;
  static constexpr int TMEM_COLS = 512;  // 2 x 128 (Z) + N2
  static_assert(K1 % 64 == 0 && K1 >= 64 && K1 <= 512, "K1");
  static_assert(N2 == 128 || N2 == 256, "N2");
  static_assert(NSLOT >= CI + TI, "ring too small");
  static_assert(512 + (2 * NSLOT + 2 * NREADY + 14) * 8 + 16 <= AUX_BYTES, "barrier area");
};

template <class Cfg>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg::NTHREADS, 1)
chain_pair_sm100_kernel(const __grid_constant__ CUtensorMap tmR, const __grid_constant__ CUtensorMap tmC,
                        const __grid_constant__ CUtensorMap tmT, const __grid_constant__ CUtensorMap tmO,
                        const ChainParams p) {
  constexpr int K1B = Cfg::K1B, N2 = Cfg::N2, NSLOT = Cfg::NSLOT, MODE = Cfg::MODE, NREADY = Cfg::NREADY;
  constexpr int CI = Cfg::CI, TI = Cfg::TI, ITEM = Cfg::ITEM_BYTES;
  constexpr bool GENERAL = Cfg::GENERAL, BF16 = Cfg::BF16;
  constexpr int CBOX = Cfg::CBOX_BYTES, TBOX = Cfg::TBOX_BYTES;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sR = smem;
  uint8_t* sRing = smem + Cfg::R_BYTES;
  float* rs = reinterpret_cast<float*>(sRing + NSLOT * ITEM);  // [128] row sums of the finished item (forward)
  uint64_t* bars = reinterpret_cast<uint64_t*>(rs + 128);
  // "own": used in both CTAs for their own data. "leader": only the leader's copy is used; threads of both
  // CTAs arrive on it.
  uint64_t* r_full = bars;                    // own    [1] resident tile landed (transaction count)
  uint64_t* slot_full = bars + 1;             // own    [NSLOT]
  uint64_t* slot_empty = slot_full + NSLOT;   // own    [NSLOT] slot may be refilled (commit from the leader, or the own epilogue)
  uint64_t* z_full = slot_empty + NSLOT;      // own    [2] GEMM1 of a block complete
  uint64_t* w_full = z_full + 2;              // leader [2] W written by the 512 element-wise threads of the pair
  uint64_t* acc_done = w_full + 2;            // own    [1] GEMM2 of a work item complete
  uint64_t* acc_free = acc_done + 1;          // leader [1] accumulators drained by the 256 epilogue threads
  uint64_t* r_free = acc_free + 1;            // own    [1] GEMM1 of a work item complete: R may be overwritten
  uint64_t* z_free = r_free + 1;              // leader [2] GEMM2 of a block complete: its Z/W buffer may be rewritten
  uint64_t* r_ready = z_free + 2;             // leader [1] resident tiles of both CTAs landed (2 arrivals)
  uint64_t* rs_free = r_ready + 1;            // own    [1] forward: row sums consumed by the own epilogue (128 arrivals)
  uint64_t* c_ready = rs_free + 1;            // leader [NREADY] a C operand group landed in both CTAs (2 arrivals)
  uint64_t* t_ready = c_ready + NREADY;       // leader [NREADY] same for a T tile
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(t_ready + NREADY);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int cluster_id = blockIdx.x >> 1;
  const int n_clusters = gridDim.x >> 1;
  // Items are numbered  w = (bh * ny + chunk) * nrb + k,  256-row block = k-th heaviest  (nrb counts 256-row blocks
  // here); see decode_step below for the order in which a cluster of the persistent grid takes them.
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
  // Work list of a cluster. With the blocks above the diagonal skipped the k-th heaviest and the k-th lightest row
  // block of a slice together always cost the same number of blocks, so the list is made of such pairs
  // ("super-items", heavy one first) and handed out round-robin: every cluster gets the same work up to one
  // super-item, whatever the number of clusters. (Single items handed out round-robin left the most loaded cluster
  // about 10 % above the mean at 2048 rows.) Step u of a cluster: super-item s = cluster + n_clusters * (u / 2),
  // first or second member.
  const int npair = (p.nrb + 1) / 2;
  const int n_super = (p.total_items / p.nrb) * npair;
  const int n_steps = cluster_id < n_super ? 2 * ((n_super - cluster_id + n_clusters - 1) / n_clusters) : 0;
  auto decode_step = [&](int u, ChainItem& it) -> bool {
    const int sidx = cluster_id + n_clusters * (u >> 1);
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
      mbar_init(&w_full[i], 512);
      mbar_init(&z_free[i], 1);
    }
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 256);
    mbar_init(r_free, 1);
    mbar_init(r_ready, 2);
    mbar_init(rs_free, 128);
    for (int i = 0; i < NREADY; ++i) {
      mbar_init(&c_ready[i], 2);
      mbar_init(&t_ready[i], 2);
    }
    ab->flag = 0;
    fence_mbar_init();
  }
  if (threadIdx.x < 128) rs[threadIdx.x] = 0.f;
  if (warp == 4) {
    tmem_alloc2(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish2();
  }
  if (warp == 6 && lane == 0) {
    tma_prefetch_desc(&tmR);
    tma_prefetch_desc(&tmC);
    tma_prefetch_desc(&tmT);
    tma_prefetch_desc(&tmO);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // the barriers of both CTAs exist before anyone arrives on the peer's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  // The next kernel in the stream, if it was launched as a programmatic dependent (the backward's three kernels are
  // independent of each other), may take over SMs as this kernel's CTAs exit instead of waiting for the whole grid.
  pdl_launch_dependents();
  const uint32_t tZ0 = tmem_base;          // Z buffers at columns [0,128) and [128,256); W overlays [0,32) and [64,96)
  const uint32_t tACC = tmem_base + 256;   // [256, 256+N2)
  // leader's copies of the shared barriers, as shared::cluster addresses usable from both CTAs
  const uint32_t l_w_full = mapa_shared(smem_u32(w_full), 0);
  const uint32_t l_acc_free = mapa_shared(smem_u32(acc_free), 0);
  const uint32_t l_c_ready = mapa_shared(smem_u32(c_ready), 0);
  const uint32_t l_t_ready = mapa_shared(smem_u32(t_ready), 0);
  const uint32_t l_r_ready = mapa_shared(smem_u32(r_ready), 0);

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
      for (int u = 0; u < n_steps && ok; ++u) {
        ChainItem it;
        if (!decode_step(u, it) || it.n_iter == 0) continue;
        // the resident tile may be overwritten once GEMM1 of the previous item has completed
        if (kacc > 0) ok = mbar_wait(r_free, (kacc - 1) & 1, ab, kCtRFree);
        if (!ok) break;
        AB200_CTR(1, kacc, 4);
        mbar_expect_tx(r_full, Cfg::R_BYTES);
#pragma unroll
        for (int c = 0; c < K1B; ++c) tma_load_3d(sR + c * TBOX, &tmR, r_full, c * 64, it.row0 + rank * 128, it.bh);
        ++kacc;
        if (u + 1 < n_steps) {
          // the next item's resident tile usually comes from HBM: ask the L2 for it now
          ChainItem nx;
          if (decode_step(u + 1, nx) && nx.n_iter > 0) {
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
              const int nb = (K1B - 2 * i) >= 2 ? 2 : 1;
              mbar_expect_tx(&slot_full[slot], nb * CBOX);
              for (int b = 0; b < nb; ++b)
                tma_load_3d(sRing + slot * ITEM + b * CBOX, &tmC, &slot_full[slot], (2 * i + b) * 64,
                            (it.t_start + t) * 128 + rank * 64, it.bh);
              ++bi;
            }
          }
          if (t >= 1) {
            for (int j = 0; j < TI && ok; ++j) {
              const int slot = acquire();
              if (!ok) break;
              mbar_expect_tx(&slot_full[slot], TBOX);
              tma_load_3d(sRing + slot * ITEM, &tmT, &slot_full[slot], it.n_off + j * 128 + rank * 64,
                          (it.t_start + t - 1) * 128, it.bh);
              ++bi;
            }
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
    // Walks the ring in order, waits for every own item to land and arrives once per operand group (up to two
    // items) on the leader's ready barrier, which completes when both CTAs have arrived.
    bool ok = true;
    int bi = 0;
    int cg = 0, tg = 0, kacc = 0;
    auto post = [&](int nitems, uint32_t ready_base, int& counter) {
      for (int i0 = 0; i0 < nitems && ok; i0 += 2) {
        for (int i = i0; i < nitems && i < i0 + 2 && ok; ++i, ++bi)
          ok = mbar_wait_warp(&slot_full[bi % NSLOT], (bi / NSLOT) & 1, ab, kCtSlotFull);
        if (ok && elect_one()) mbar_arrive_cluster(ready_base + (counter % NREADY) * 8);
        __syncwarp();
        ++counter;
      }
    };
    for (int u = 0; u < n_steps && ok; ++u) {
      ChainItem it;
      if (!decode_step(u, it)) continue;
      const int n = it.n_iter;
      if (n == 0) continue;
      ok = mbar_wait_warp(r_full, kacc & 1, ab, kCtR);
      if (lane == 0) AB200_CTR(1, kacc, 5);
      if (ok && elect_one()) mbar_arrive_cluster(l_r_ready);
      __syncwarp();
      ++kacc;
      for (int t = 0; t <= n && ok; ++t) {
        if (t < n) post(CI, l_c_ready, cg);
        if (t >= 1) post(TI, l_t_ready, tg);
      }
    }
  } else if ((warp == 4 || warp == 5) && rank == 0) {
    // ------------------------------------------------------------------ MMA issuers (leader CTA only)
    // Warp 4 issues GEMM1 (Z), warp 5 GEMM2 (ACC); converged warps, one elected lane issues. Ring items are
    // consumed in a fixed order:  C_0 at b0;  C_t at b0 + CI + (t-1)(CI+TI);  T_t right after C_{t+1}, except
    // the last T_{n-1}, which follows T_{n-2} directly. Both CTAs keep identical rings, so one slot index
    // addresses the operand halves of both.
    constexpr uint32_t idesc_z = umma_idesc(256, 128, BF16, false, false);
    constexpr uint32_t idesc_acc = umma_idesc(256, 128, BF16, false, true);
    bool ok = true;
    int b0 = 0;    // ring items of earlier work items
    int g0 = 0;    // 128-wide blocks of earlier work items (selects Z buffer and ready barrier)
    int kacc = 0;  // non-empty work items finished so far
    int cg = 0, tg = 0;  // operand groups consumed so far (as the scouts count them)
    const uint32_t r_addr = smem_u32(sR);
    const uint32_t ring_addr = smem_u32(sRing);
    for (int u = 0; u < n_steps && ok; ++u) {
      ChainItem it;
      if (!decode_step(u, it)) continue;
      const int n = it.n_iter;
      if (n == 0) continue;
      if (warp == 4) {
        ok = mbar_wait_warp(r_ready, kacc & 1, ab, kCtR);
        if (lane == 0) AB200_CTR(1, kacc, 6);
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
            ok = mbar_wait_warp(&c_ready[cg % NREADY], (cg / NREADY) & 1, ab, kCtSlotFull);
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
                        umma_ss2(tz, umma_smem_desc(r_addr + (2 * i + b) * TBOX + ks * 32, 16, 1024),
                                 umma_smem_desc(a + b * CBOX + ks * 32, 16, 1024), idesc_z,
                                 (i > 0 || b > 0 || ks > 0) ? 1u : 0u);
                    }
                  }
                  // (the first slots of a work item's last C tile may go to the epilogues, like those of its last T tile)
                  if (!(Cfg::ONE_ROUND && t + 1 == n && i < TI)) tc_commit2_both(&slot_empty[slot]);
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
            if (lane == 0) AB200_CTR(1, kacc, 7);
          }
          ok = mbar_wait_warp(&w_full[g & 1], (g >> 1) & 1, ab, kCtWFull);
          if (!ok) break;
          if (lane == 0) AB200_CTR(1, g, 2);
          const uint32_t tw = tZ0 + (g & 1) * 128;
          const int base = b0 + CI + t * (CI + TI) + (t + 1 < n ? CI : 0);
          ok = mbar_wait_warp(&t_ready[tg % NREADY], (tg / NREADY) & 1, ab, kCtSlotFull);
          ++tg;
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
#pragma unroll
            for (int j = 0; j < TI; ++j) {
              const int slot = (base + j) % NSLOT;
              const uint32_t a = ring_addr + slot * ITEM;
#pragma unroll
              for (int ks = 0; ks < 8; ++ks)
                umma_ts2(tACC + j * 128, tw + (ks < 4 ? ks * 8 : 64 + (ks - 4) * 8), umma_smem_desc(a + ks * 2048, TBOX, 1024),
                         idesc_acc, (t > 0 || ks > 0) ? 1u : 0u);
              // the slots of the last T tile go to the epilogues (output staging), which hand them back
              if (t + 1 < n) tc_commit2_both(&slot_empty[slot]);
            }
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
  } else if (warp < 4 || (warp >= 8 && warp < 12)) {
    // ------------------------------------------------------------------ element-wise warpgroups (own 128 rows)
    // Warpgroup hh = 0 (warps 0-3) handles columns [0,64) of every block, hh = 1 (warps 8-11) columns [64,128).
    const int hh = warp >= 8 ? 1 : 0;
    const int tid = threadIdx.x & 127;  // TMEM lane = row of the CTA's tile
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    constexpr bool decay_mode = !GENERAL;
    bool ok = true;
    int g0 = 0;     // blocks processed before the current work item
    int kacc = 0;   // non-empty work items finished so far
    for (int u = 0; u < n_steps && ok; ++u) {
      ChainItem it;
      if (!decode_step(u, it)) continue;
      const int bh = it.bh, row0 = it.row0 + static_cast<int>(rank) * 128, n_off = it.n_off, t_start = it.t_start;
      const int n_iter = it.n_iter;
      const int grow = row0 + tid;  // global row index on the row side
      const int h = bh % p.H;
      float lg = 0.f;  // log2(gamma)
      if (decay_mode) lg = log2f(p.decay[h]);
      float rowf_base = p.scale;
      if (decay_mode) rowf_base *= exp2f((MODE == kChainRowK ? -tid : tid) * lg);
      if (MODE == kChainRowQ) rowf_base *= (grow < p.Lq) ? 1.0f / p.r_in[static_cast<size_t>(bh) * p.Lq + grow] : 0.f;
      float rsum = 0.f;
      if (n_iter == 0) {
        // no block contributes to this tile: zeros (and r = 1 in the forward)
        if (hh == 0 && grow < rows_len) {
          uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * rows_len + grow) * p.ld_out + n_off;
          for (int c = 0; c < N2; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
          if (MODE == kChainFwd && n_off == 0) p.r_out[static_cast<size_t>(bh) * p.Lq + grow] = 1.0f;
        }
        continue;
      }

      for (int t = 0; t < n_iter; ++t) {
        const int g = g0 + t;  // running block index: Z buffer g & 1
        const int col0 = (t_start + t) * 128;
        float colf0 = 0.f, colf1 = 0.f;
        if (MODE == kChainRowK) {
          // column factor gamma^c / r[c] (decay) or 1 / r[c] (mask tensor: lg = 0) of column (chunk, lane)
          colf0 = chain_rowk_colf(p, bh, col0, 2 * hh, lane, lg);
          colf1 = chain_rowk_colf(p, bh, col0, 2 * hh + 1, lane, lg);
        }
        uint32_t mk[GENERAL ? 32 : 1];
        if constexpr (GENERAL && MODE != kChainRowK) {
          // the block's mask values of this thread (its row of the mask tensor), fetched before the wait for Z
          if (hh == 0) chain_mask_prefetch<MODE, 0>(p, h, grow, col0, mk);
          else chain_mask_prefetch<MODE, 2>(p, h, grow, col0, mk);
        } else if constexpr (GENERAL) {
          // RowK: the thread's column of the mask, read by rows by the whole warp and transposed in registers
          if (p.mask_t != nullptr) {  // a transposed copy of the mask exists: the thread's column is a row of it
            if (hh == 0) chain_mask_prefetch_t<0>(p, h, grow, col0, mk);
            else chain_mask_prefetch_t<2>(p, h, grow, col0, mk);
          } else if (hh == 0) {
            chain_mask_prefetch_rowk<0>(p, h, grow - lane, lane, col0, mk);
          } else {
            chain_mask_prefetch_rowk<2>(p, h, grow - lane, lane, col0, mk);
          }
        }
        float rowf = rowf_base;
        if (decay_mode) rowf *= exp2f((MODE == kChainRowK ? (col0 - row0) : (row0 - col0)) * lg);
        //   Fwd/RowQ: column c valid iff col0 + c <= grow ;  RowK: valid iff col0 + c >= grow
        const bool straddle = decay_mode && (MODE == kChainRowK ? (col0 < row0 + 127) : (col0 + 127 > row0));
        const int dlim = grow - col0;

        if (tid == 0 && hh == 0) AB200_CTR(0, g, 0);
        ok = mbar_wait_warp(&z_full[g & 1], (g >> 1) & 1, ab, kCtZFull);
        if (!ok) break;
        if (tid == 0 && hh == 0) AB200_CTR(0, g, 1);
        tc_fence_after();
        const uint32_t tz = tmem_addr(tZ0 + (g & 1) * 128, lane_base, 0);
        if constexpr (GENERAL) {
          if (hh == 0) chain_ew_mask2<MODE, BF16, 0, true>(tz, mk, rowf, colf0, colf1, rsum);
          else chain_ew_mask2<MODE, BF16, 2, true>(tz, mk, rowf, colf0, colf1, rsum);
        } else {
          if (hh == 0) chain_ew_decay2<MODE, BF16, 0, true>(tz, rowf, lg, colf0, colf1, straddle, dlim, rsum);
          else chain_ew_decay2<MODE, BF16, 2, true>(tz, rowf, lg, colf0, colf1, straddle, dlim, rsum);
        }
        if (MODE == kChainFwd && t + 1 == n_iter) {
          // both halves add their partial row sums into the (zeroed) buffer the own epilogue reads; it must have
          // consumed the previous item's sums
          if (kacc > 0) {
            ok = mbar_wait_warp(rs_free, (kacc - 1) & 1, ab, kCtAccFree);
            if (!ok) break;
          }
          atomicAdd(&rs[tid], rsum);
        }
        if (tid == 0 && hh == 0) AB200_CTR(0, g, 2);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive_cluster(l_w_full + (g & 1) * 8);
        if (tid == 0 && hh == 0) AB200_CTR(0, g, 3);
      }
      if (!ok) break;
      g0 += n_iter;
      ++kacc;
    }
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ epilogue warpgroup (own 128 rows)
    // ACC -> scale -> 16-bit -> shared memory (128-byte swizzle, 64-column boxes) -> TMA store, in two rounds of
    // TI boxes staged in the ring slots of the work item's last T tile.
    const int tid = threadIdx.x - 384;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32);
    bool ok = true;
    int kacc = 0;
    int b0 = 0;
    for (int u = 0; u < n_steps && ok; ++u) {
      ChainItem it;
      if (!decode_step(u, it)) continue;
      const int n = it.n_iter;
      if (n == 0) continue;  // warpgroup A writes the zeros of an empty tile
      const int row0 = it.row0 + static_cast<int>(rank) * 128;
      const int grow = row0 + tid;
      const int tbase = b0 + CI + (n - 1) * (CI + TI);  // ring index of the first item of the last T tile
      ok = mbar_wait_warp(acc_done, kacc & 1, ab, kCtAccDone);
      if (!ok) break;
      if (tid == 0) AB200_CTR(0, kacc, 4);
      tc_fence_after();
      float osc = 1.0f;
      if (MODE == kChainFwd) {
        const float r = fmaxf(rs[tid], 1.0f);
        rs[tid] = 0.f;
        mbar_arrive(rs_free);
        osc = 1.0f / r;
        if (it.n_off == 0 && grow < rows_len) p.r_out[static_cast<size_t>(it.bh) * p.Lq + grow] = r;
      }
      const uint32_t ta = tmem_addr(tACC, lane_base, 0);
      constexpr int NROUND = Cfg::ONE_ROUND ? 1 : 2;
      constexpr int NBOX = 2 * TI / NROUND;  // 64-column boxes staged per round
      const int cbase = b0 + (n == 1 ? 0 : CI + (n - 2) * (CI + TI));  // ring index of the first item of the last C tile
      auto stage_slot = [&](int j) -> int { return ((j < TI ? tbase + j : cbase + (j - TI)) % NSLOT); };
#pragma unroll
      for (int round = 0; round < NROUND; ++round) {
        if (round == 1) {
          // the stores of pass 0 must have read the staging slots before they are overwritten
          if (tid == 0) tma_store_wait_read0();
          asm volatile("bar.sync 3, 128;" ::: "memory");
        }
#pragma unroll
        for (int j = 0; j < NBOX; ++j) {
          const int box = round * NBOX + j;
          uint8_t* stage = sRing + stage_slot(j) * ITEM + tid * 128;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t rr[32];
            tmem_ld32(ta + box * 64 + half * 32, rr);
            tc_wait_ld();
            if (round == NROUND - 1 && j == NBOX - 1 && half == 1) {
              // every column of the accumulator is in registers now: GEMM2 of the next item may overwrite it
              tc_fence_before();
              mbar_arrive_cluster(l_acc_free);
              if (tid == 0) AB200_CTR(0, kacc, 5);
            }
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 v;
              v.x = pack2<BF16>(__uint_as_float(rr[q4 * 8 + 0]) * osc, __uint_as_float(rr[q4 * 8 + 1]) * osc);
              v.y = pack2<BF16>(__uint_as_float(rr[q4 * 8 + 2]) * osc, __uint_as_float(rr[q4 * 8 + 3]) * osc);
              v.z = pack2<BF16>(__uint_as_float(rr[q4 * 8 + 4]) * osc, __uint_as_float(rr[q4 * 8 + 5]) * osc);
              v.w = pack2<BF16>(__uint_as_float(rr[q4 * 8 + 6]) * osc, __uint_as_float(rr[q4 * 8 + 7]) * osc);
              const int chunk = half * 4 + q4;  // 16-byte chunk of the 128-byte row, XOR-swizzled by the row
              *reinterpret_cast<uint4*>(stage + ((chunk ^ (tid & 7)) << 4)) = v;
            }
          }
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 3, 128;" ::: "memory");
        if (tid == 0 && row0 < rows_len) {  // rows past the end of the tensor are clipped by the store; a tile that lies
                                            // wholly outside is not stored at all
#pragma unroll
          for (int j = 0; j < NBOX; ++j)
            tma_store_3d(&tmO, sRing + stage_slot(j) * ITEM, it.n_off + (round * NBOX + j) * 64, row0, it.bh);
          tma_store_commit();
        }
      }
      if (tid == 0) {
        // hand the staging slots back to the producer once the stores have read them
        tma_store_wait_read0();
#pragma unroll
        for (int j = 0; j < NBOX; ++j) mbar_arrive(&slot_empty[stage_slot(j)]);
        AB200_CTR(0, kacc, 6);
      }
      b0 += n * (CI + TI);
      ++kacc;
    }
    if (tid == 0) tma_store_wait0();  // all output written before the CTA exits
  }

  __syncwarp();
  // A programmatic dependent must not complete before the kernel it overlapped with: completion then stays
  // ordered along the stream for whatever comes next.
  if (threadIdx.x == 0) pdl_grid_dependency_wait();
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // no CTA leaves while the other may still arrive on its barriers or its MMAs read this CTA's memory
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
