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
// Roles: warps 0-3 element-wise warpgroup (thread t owns TMEM lane t), warp 4 issues every tcgen05.mma
// (converged warp, one elected lane), warp 5 lane 0 is the TMA producer. Z is double buffered in tensor
// memory so that GEMM1 of block t+1 runs while the warpgroup works on block t. All streamed operands
// travel through one ring of 32 KB items (two boxes of 128 rows x 64 columns, 128-byte swizzle).
#pragma once

#include "ptx.cuh"

namespace ab200 {

enum ChainMode : int { kChainFwd = 0, kChainRowQ = 1, kChainRowK = 2 };

struct ChainParams {
  void* out;             // [BH, rows, ld_out] 16-bit; this CTA writes columns [z*N2, z*N2+N2)
  int ld_out;
  float* r_out;          // Fwd: [BH, Lq] normaliser r = max(sum_j |S~|, 1), written by z == 0
  const float* r_in;     // RowQ / RowK: [BH, Lq]
  const uint16_t* mask;  // general mask [H, Lq, Lkv] (16-bit, same dtype as the operands) or nullptr
  const float* decay;    // per-head gamma [H] or nullptr (exactly one of mask / decay is set)
  int H, Lq, Lkv;
  float scale;
  int skip_upper;        // 1: blocks strictly above the diagonal are all zero and are skipped
};

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
  static constexpr int NTHREADS = 192;  // element-wise warpgroup + MMA issuer warp + TMA producer warp
  static constexpr int TMEM_COLS = 512;  // 2 x 128 (Z) + N2
  static_assert(K1 % 64 == 0 && K1 >= 64 && K1 <= 512, "K1");
  static_assert(N2 % 64 == 0 && N2 >= 64 && N2 <= 256, "N2");
  static_assert(NSLOT >= 3, "ring too small");
  static_assert(2 * NSLOT + 8 <= 64, "barrier area");
};

// Optional event trace (compile with -DAB200_TRACE), see fa_fwd_sm100.cuh: CTA (0,0,0) only.
#ifdef AB200_TRACE
constexpr int kChainTraceIters = 16;
__device__ long long g_chain_trace[2][kChainTraceIters][8];
#define AB200_CTR(who, j, ev)                                                                            \
  do {                                                                                                   \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < kChainTraceIters) g_chain_trace[who][j][ev] = clock64(); \
  } while (0)
#else
#define AB200_CTR(who, j, ev) do {} while (0)
#endif

enum ChainTag : int { kCtR = 11, kCtSlotFull = 12, kCtSlotEmpty = 13, kCtZFull = 14, kCtWFull = 15, kCtAccDone = 16 };

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
  float* cf = reinterpret_cast<float*>(sRing + NSLOT * ITEM);  // [2][128] column factors
  uint64_t* bars = reinterpret_cast<uint64_t*>(cf + 256);
  uint64_t* r_full = bars;                    // [1]
  uint64_t* slot_full = bars + 1;             // [NSLOT]
  uint64_t* slot_empty = slot_full + NSLOT;   // [NSLOT]
  uint64_t* z_full = slot_empty + NSLOT;      // [2]
  uint64_t* w_full = z_full + 2;              // [2]
  uint64_t* acc_done = w_full + 2;            // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);  // provably warp-uniform
  const int lane = threadIdx.x & 31;
  // grid: x = row block, y = column chunk, z = (batch, head): the chunks of one slice run side by side and
  // share their streamed operands in L2
  const int bh = blockIdx.z;
  const int n_off = blockIdx.y * N2;

  // row side = the resident tile; column side = the streamed blocks
  const int rows_len = (MODE == kChainRowK) ? p.Lkv : p.Lq;
  const int cols_len = (MODE == kChainRowK) ? p.Lq : p.Lkv;
  const int nrb = (rows_len + 127) / 128;
  // heaviest row blocks first when blocks are skipped (Fwd/RowQ: late queries; RowK: early keys)
  const int rb = (p.skip_upper && MODE != kChainRowK) ? (nrb - 1 - blockIdx.x) : blockIdx.x;
  const int row0 = rb * 128;
  const int ncb = (cols_len + 127) / 128;
  int t_start = 0, n_iter = ncb;
  if (p.skip_upper) {
    if (MODE == kChainRowK) {
      t_start = row0 / 128;  // query blocks that end before this key block see none of its keys
      n_iter = ncb - t_start;
    } else {
      const int last = row0 / 128 + 1;  // key blocks up to the one containing the last query row
      n_iter = last < ncb ? last : ncb;
    }
    if (n_iter < 0) n_iter = 0;
  }

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
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 5 && lane == 0) {
    tma_prefetch_desc(&tmR);
    tma_prefetch_desc(&tmC);
    tma_prefetch_desc(&tmT);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const uint32_t tZ0 = tmem_base;          // Z buffers at columns [0,128) and [128,256); W overlays the first 64
  const uint32_t tACC = tmem_base + 256;   // [256, 256+N2)

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_iter > 0) {
      bool ok = true;
      mbar_expect_tx(r_full, Cfg::R_BYTES);
#pragma unroll
      for (int c = 0; c < K1B; ++c) tma_load_3d(sR + c * BOX, &tmR, r_full, c * 64, row0, bh);
      int bi = 0;  // items issued
      // one item = boxes [2i, 2i+2) of the tile (the last item of an odd tile holds one box)
      auto put = [&](const CUtensorMap* map, int x0, int nboxes, int y) {
        const int slot = bi % NSLOT;
        const int use = bi / NSLOT;
        if (use > 0) ok = mbar_wait(&slot_empty[slot], (use - 1) & 1, ab, kCtSlotEmpty);
        if (!ok) return;
        mbar_expect_tx(&slot_full[slot], nboxes * BOX);
        for (int b = 0; b < nboxes; ++b)
          tma_load_3d(sRing + slot * ITEM + b * BOX, map, &slot_full[slot], x0 + b * 64, y, bh);
        ++bi;
      };
      // consumption order: C_0, then for t >= 1: C_t, T_{t-1}; finally T_{n-1}
      for (int t = 0; t <= n_iter && ok; ++t) {
        if (t < n_iter) {
          for (int i = 0; i < CI && ok; ++i)
            put(&tmC, i * 128, (K1B - 2 * i) >= 2 ? 2 : 1, (t_start + t) * 128);
        }
        if (t >= 1) {
          for (int i = 0; i < TI && ok; ++i)
            put(&tmT, n_off + i * 128, (N2B - 2 * i) >= 2 ? 2 : 1, (t_start + t - 1) * 128);
        }
      }
      if (!ok) {
        mbar_wait_drain(r_full, 0, 2000000ull);
        for (int slot = 0; slot < NSLOT; ++slot)
          if (bi > slot) mbar_wait_drain(&slot_full[slot], ((bi - 1 - slot) / NSLOT) & 1, 2000000ull);
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp runs converged (waits included) and one elected lane issues, so that addresses and
    // descriptors stay warp-uniform. (Splitting GEMM1 and GEMM2 over two issuing warps was measured and
    // does not pay: the kernel is bound by the L2->SM operand stream, not by issue slots.)
    if (n_iter > 0) {
      constexpr uint32_t idesc_z = umma_idesc(128, 128, BF16, false, false);
      constexpr uint32_t idesc_acc2 = umma_idesc(128, 128, BF16, false, true);  // two boxes: N = 128
      constexpr uint32_t idesc_acc1 = umma_idesc(128, 64, BF16, false, true);   // one box:   N = 64
      bool ok = true;
      int bi = 0;  // items consumed
      auto take = [&](int& slot) -> uint32_t {
        slot = bi % NSLOT;
        ok = mbar_wait_warp(&slot_full[slot], (bi / NSLOT) & 1, ab, kCtSlotFull);
        ++bi;
        return smem_u32(sRing) + slot * ITEM;
      };
      const uint32_t r_addr = smem_u32(sR);
      auto issue_z = [&](int t) {
        const uint32_t tz = tZ0 + (t & 1) * 128;
#pragma unroll
        for (int i = 0; i < CI; ++i) {
          int slot;
          const uint32_t a = take(slot);
          if (!ok) return;
          const int nb = (K1B - 2 * i) >= 2 ? 2 : 1;
          if (elect_one()) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              if (b < nb) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks)
                  umma_ss(tz, umma_smem_desc(r_addr + (2 * i + b) * BOX + ks * 32, 16, 1024),
                          umma_smem_desc(a + b * BOX + ks * 32, 16, 1024), idesc_z, (i > 0 || b > 0 || ks > 0) ? 1u : 0u);
              }
            }
            tc_commit(&slot_empty[slot]);
            if (i == CI - 1) tc_commit(&z_full[t & 1]);
          }
          __syncwarp();
        }
      };
      auto issue_acc = [&](int t) {
        ok = mbar_wait_warp(&w_full[t & 1], (t >> 1) & 1, ab, kCtWFull);
        if (!ok) return;
        if (lane == 0) AB200_CTR(1, t, 2);
        tc_fence_after();
        const uint32_t tw = tZ0 + (t & 1) * 128;
#pragma unroll
        for (int i = 0; i < TI; ++i) {
          int slot;
          const uint32_t a = take(slot);
          if (!ok) return;
          const bool two = (N2B - 2 * i) >= 2;
          if (elect_one()) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              umma_ts(tACC + i * 128, tw + ks * 8, umma_smem_desc(a + ks * 2048, BOX, 1024), two ? idesc_acc2 : idesc_acc1,
                      (t > 0 || ks > 0) ? 1u : 0u);
            tc_commit(&slot_empty[slot]);
            if (i == TI - 1 && t == n_iter - 1) tc_commit(acc_done);
          }
          __syncwarp();
        }
      };
      ok = mbar_wait_warp(r_full, 0, ab, kCtR);
      if (ok) {
        tc_fence_after();
        issue_z(0);
        for (int t = 0; t < n_iter && ok; ++t) {
          if (lane == 0) AB200_CTR(1, t, 0);
          if (t + 1 < n_iter) issue_z(t + 1);
          if (lane == 0) AB200_CTR(1, t, 1);
          if (ok) issue_acc(t);
          if (lane == 0) AB200_CTR(1, t, 3);
        }
      }
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ element-wise warpgroup
    const int tid = threadIdx.x;  // 0..127 = TMEM lane = row of the resident tile
    const int grow = row0 + tid;  // global row index on the row side
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32);
    const int h = bh % p.H;
    const bool decay_mode = !GENERAL;
    float lg = 0.f;  // log2(gamma)
    if (decay_mode) lg = log2f(p.decay[h]);
    // per-row factor that does not depend on the block
    float rowf_base = p.scale;
    if (decay_mode) rowf_base *= exp2f((MODE == kChainRowK ? -tid : tid) * lg);
    if (MODE == kChainRowQ) rowf_base *= (grow < p.Lq) ? 1.0f / p.r_in[static_cast<size_t>(bh) * p.Lq + grow] : 0.f;
    if (MODE != kChainRowK && decay_mode) {
      cf[tid] = exp2f(-tid * lg);  // gamma^(-c)
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    float rsum = 0.f;
    bool ok = true;

    for (int t = 0; t < n_iter; ++t) {
      const int col0 = (t_start + t) * 128;
      const float* cft = cf;
      if (MODE == kChainRowK) {
        // column factor: 1/r of the block's queries (times gamma^c under decay)
        const int qi = col0 + tid;
        float f = (qi < p.Lq) ? 1.0f / p.r_in[static_cast<size_t>(bh) * p.Lq + qi] : 0.f;
        if (decay_mode) f *= exp2f(tid * lg);
        cf[(t & 1) * 128 + tid] = f;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        cft = cf + (t & 1) * 128;
      }
      float rowf = rowf_base;
      if (decay_mode) rowf *= exp2f((MODE == kChainRowK ? (col0 - row0) : (row0 - col0)) * lg);
      // triangular predicate only on blocks that straddle the diagonal (decay mode)
      //   Fwd/RowQ: column c valid iff col0 + c <= grow ;  RowK: valid iff col0 + c >= grow
      const bool straddle = decay_mode && (MODE == kChainRowK ? (col0 < row0 + 127) : (col0 + 127 > row0));
      const int dlim = grow - col0;

      if (tid == 0) AB200_CTR(0, t, 0);
      ok = mbar_wait_warp(&z_full[t & 1], (t >> 1) & 1, ab, kCtZFull);
      if (!ok) break;
      if (tid == 0) AB200_CTR(0, t, 1);
      tc_fence_after();
      const uint32_t tz = tmem_addr(tZ0 + (t & 1) * 128, lane_base, 0);
#pragma unroll
      for (int qd = 0; qd < 4; ++qd) {
        uint32_t zr[32];
        tmem_ld32(tz + qd * 32, zr);
        float mk[32];
        if (GENERAL) {
          if (MODE != kChainRowK) {
            // row of the mask owned by this thread: M[h, grow, col0 + qd*32 ...], 16-byte vectors
            const uint16_t* mp = p.mask + (static_cast<size_t>(h) * p.Lq + grow) * p.Lkv + col0 + qd * 32;
#pragma unroll
            for (int v8 = 0; v8 < 4; ++v8) {
              uint4 u = make_uint4(0, 0, 0, 0);
              if (grow < p.Lq && col0 + qd * 32 + v8 * 8 < p.Lkv) u = __ldg(reinterpret_cast<const uint4*>(mp) + v8);
              const uint32_t w4[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if constexpr (BF16) {
                  mk[v8 * 8 + 2 * e] = __uint_as_float(w4[e] << 16);
                  mk[v8 * 8 + 2 * e + 1] = __uint_as_float(w4[e] & 0xffff0000u);
                } else {
                  const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&w4[e]));
                  mk[v8 * 8 + 2 * e] = f2.x;
                  mk[v8 * 8 + 2 * e + 1] = f2.y;
                }
              }
            }
          } else {
            // column of the mask: M[h, col0 + c, grow]; consecutive threads read consecutive keys
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              const int qi = col0 + qd * 32 + c;
              uint16_t u = 0;
              if (qi < p.Lq && grow < p.Lkv) u = __ldg(p.mask + (static_cast<size_t>(h) * p.Lq + qi) * p.Lkv + grow);
              if constexpr (BF16) {
                mk[c] = __uint_as_float(static_cast<uint32_t>(u) << 16);
              } else {
                mk[c] = __half2float(__ushort_as_half(u));
              }
            }
          }
        }
        tc_wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          float w0 = __uint_as_float(zr[c]) * rowf;
          float w1 = __uint_as_float(zr[c + 1]) * rowf;
          if (GENERAL) {
            w0 *= mk[c];
            w1 *= mk[c + 1];
          }
          if (MODE == kChainRowK || decay_mode) {
            w0 *= cft[qd * 32 + c];
            w1 *= cft[qd * 32 + c + 1];
          }
          if (straddle) {
            const int cc = qd * 32 + c;
            if (MODE == kChainRowK) {
              if (cc < dlim) w0 = 0.f;
              if (cc + 1 < dlim) w1 = 0.f;
            } else {
              if (cc > dlim) w0 = 0.f;
              if (cc + 1 > dlim) w1 = 0.f;
            }
          }
          if (MODE == kChainFwd) rsum += fabsf(w0) + fabsf(w1);
          pk[c >> 1] = pack2<BF16>(w0, w1);
        }
        tmem_st16(tz + qd * 16, pk);
      }
      if (tid == 0) AB200_CTR(0, t, 2);
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(&w_full[t & 1]);
      if (tid == 0) AB200_CTR(0, t, 3);
    }

    // ---- epilogue
    uint16_t* orow = reinterpret_cast<uint16_t*>(p.out) + (static_cast<size_t>(bh) * rows_len + grow) * p.ld_out + n_off;
    if (ok && n_iter > 0) {
      ok = mbar_wait_warp(acc_done, 0, ab, kCtAccDone);
      if (ok) {
        tc_fence_after();
        float osc = 1.0f;
        if (MODE == kChainFwd) {
          const float r = fmaxf(rsum, 1.0f);
          osc = 1.0f / r;
          if (n_off == 0 && grow < rows_len) p.r_out[static_cast<size_t>(bh) * p.Lq + grow] = r;
        }
        const uint32_t ta = tmem_addr(tACC, lane_base, 0);
#pragma unroll
        for (int c0 = 0; c0 < N2; c0 += 32) {
          uint32_t rr[32];
          tmem_ld32(ta + c0, rr);
          tc_wait_ld();
          if (grow < rows_len) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              v.x = pack2<BF16>(__uint_as_float(rr[i + 0]) * osc, __uint_as_float(rr[i + 1]) * osc);
              v.y = pack2<BF16>(__uint_as_float(rr[i + 2]) * osc, __uint_as_float(rr[i + 3]) * osc);
              v.z = pack2<BF16>(__uint_as_float(rr[i + 4]) * osc, __uint_as_float(rr[i + 5]) * osc);
              v.w = pack2<BF16>(__uint_as_float(rr[i + 6]) * osc, __uint_as_float(rr[i + 7]) * osc);
              *reinterpret_cast<uint4*>(orow + c0 + i) = v;
            }
          }
        }
      }
    } else if (ok && grow < rows_len) {
      // no block contributes to this tile: zeros (and r = 1 in the forward)
      for (int c = 0; c < N2; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
      if (MODE == kChainFwd && n_off == 0) p.r_out[static_cast<size_t>(bh) * p.Lq + grow] = 1.0f;
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

}  // namespace ab200
