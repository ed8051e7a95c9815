// Chunkwise (recurrent-state) RetNet forward for sm_100a: the unnormalised retention
//
//     O[i] = scale * sum_{j <= i} gamma^(i-j) (q_i . k_j) v_j
//
// computed in chunks of 128 positions with a running state instead of over all (i, j) pairs, so the work grows
// with L, not L^2. It is the function the reference's recurrent kernel computes with an fp32 CUB scan
// (csrc/kernels/retnet/recurrent/recurrent.h:110-114 scan operator, :132-395 scan_fwd_kernel, C entry
// retnet_recurrent_fwd :427-463: state_t = decay_t * state_{t-1} + k_t v_t^T, out_t = q_t . state_t) for a per-head
// constant decay, and the "chunkwise retnet" its README lists as to do (README.md:103). Here the state lives in
// tensor memory and every product runs on the tcgen05 tensor cores.
//
// One CTA owns one (batch, head) slice and DVC columns of V / O and walks the sequence chunk by chunk. With
// S = state after the previous chunk [dqk x DVC] and g = gamma^128:
//
//     Z   = Q_c K_c^T                             [128 x 128]   both operands K-major in shared memory
//     ACC = Q_c S                                 [128 x DVC]   S as 16-bit copy in shared memory (MN-major B operand)
//     ACC[i] *= gamma^(i+1)                       in tensor memory, by the thread that owns row i
//     W   = Z .* gamma^(i-j) for j <= i, else 0   fp32 in registers, 16-bit written over Z in tensor memory
//     K_c[j] *= gamma^(127-j)                     in place in shared memory, once Q K^T has read the plain tile
//     S   = g S + K_c^T V_c                       fp32 in tensor memory; K_c^T (scaled rows) is the MN-major A operand
//     ACC += W V_c                                W from tensor memory
//     O_c = scale * ACC
//
// Every decay factor is applied where its value is at most 1 and in fp32 or on a term whose weight it is: W carries
// gamma^(i-j) computed in fp32 registers, the carried term is scaled in the fp32 accumulator, and the scaled K rows
// only feed the state update, where a row that underflows in 16 bits is a contribution that small. Scaling K (not V)
// lets the state update start right after Q K^T instead of after W V, so the state copy for the next chunk and the
// release of the K and V buffers come early and the next chunk's loads run under this chunk's epilogue. So no
// intermediate exceeds the magnitudes of Q K^T and V whatever gamma in (0, 1] is, and no scratch memory is needed.
//
// Roles: warps 0-3 row warpgroup (thread t owns TMEM lane t: row t of Z / ACC; W, the carried term, the output),
// warps 4-7 state warpgroup (row t of each state half and a share of the K tile; the two groups work side by side, which
// takes the scaling of K and the copy of the state off the chain Z -> W -> W V), warp 8 issues every MMA (converged
// warp, one elected lane; a single issuer keeps all tensor-memory hazards in program order), warp 9 lane 0 is the TMA
// producer. Tensor memory: Z at [0,128), ACC at
// [128,128+DVC), the state halves (dqk rows 0-127, 128-255) at [256,256+DVC) and [384,384+DVC).
//
// Few slices, long sequences: a walk in order leaves most SMs idle (a grid of BH * dv / DVC CTAs is all the parallelism
// there is). With scratch memory the sequence is cut into segments of `seg` chunks (blockIdx.z): a first kernel
// (ret_chunk_state_sm100_kernel) computes, for every segment but the last, the state that segment alone would leave
// behind (T_g = sum_c g^(last - c) K_c'^T V_c, fp32, one tile per CTA), and this kernel starts segment g > 0 from
// S = sum_{g' < g} gamma^(128 seg (g - 1 - g')) T_g', which is the state the walk in order would have carried there.
#pragma once

#include "chain_common.cuh"

namespace ab200 {

struct RetChunkParams {
  void* o;               // [BH, L, dv] 16-bit
  const float* decay;    // [H] gammas
  int H, L, dv;
  float scale;
  float* ws;             // segment states, [BH][dv / DVC][segments - 1][dqk / 128][DVC][128] fp32; null when gridDim.z == 1
  int seg;               // chunks per segment (>= number of chunks when the sequence is walked in one piece)
};

template <int DQK_, int DVC_, bool BF16_>
struct RetChunkConfig {
  static constexpr int DQK = DQK_;    // head dimension of q, k: 128 or 256 (the state tile has 128 rows per MMA)
  static constexpr int DVC = DVC_;    // columns of V / O per CTA: 64 or 128
  static constexpr bool BF16 = BF16_;
  static constexpr int C = 128;       // chunk length
  static constexpr int NH = DQK / 128;       // state halves
  static constexpr int KB = DQK / 64;        // boxes per Q / K tile
  static constexpr int VB = DVC / 64;        // boxes per V tile
  static constexpr int BOX_BYTES = 128 * 128;
  static constexpr int QK_BYTES = KB * BOX_BYTES;
  static constexpr int V_BYTES = VB * BOX_BYTES;
  static constexpr int SB_HALF_BYTES = VB * BOX_BYTES;  // 128 state rows x DVC columns, 16-bit
  static constexpr int SMEM_TILES = 2 * QK_BYTES + V_BYTES + NH * SB_HALF_BYTES;
  static constexpr int SMEM_BYTES = 1024 + SMEM_TILES + 512;
  static constexpr int NTHREADS = 320;
  static constexpr int TMEM_COLS = 512;
  static_assert(DQK == 128 || DQK == 256, "dqk");
  static_assert(DVC == 64 || DVC == 128, "dv chunk");
  static_assert(SMEM_BYTES <= 232448, "shared memory");
};

enum RetChunkTag : int {
  kRcQ = 51, kRcK = 52, kRcV = 53, kRcQFree = 54, kRcKVFree = 55, kRcZ = 56, kRcW = 57, kRcAcc = 58, kRcAccFree = 59,
  kRcU = 60, kRcState = 61, kRcY = 62, kRcKScaled = 63, kRsFull = 64, kRsEmpty = 65, kRsScaled = 66, kRsDone = 67
};

template <class Cfg>
__global__ void __launch_bounds__(Cfg::NTHREADS, 1)
ret_chunk_sm100_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                       const RetChunkParams p) {
  constexpr int DQK = Cfg::DQK, DVC = Cfg::DVC, NH = Cfg::NH, KB = Cfg::KB, VB = Cfg::VB, BOX = Cfg::BOX_BYTES;
  constexpr bool BF16 = Cfg::BF16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::QK_BYTES;
  uint8_t* sV = sK + Cfg::QK_BYTES;
  uint8_t* sSb = sV + Cfg::V_BYTES;  // NH halves of [128 state rows][DVC] 16-bit, laid out like a V tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::SMEM_TILES);
  uint64_t* q_full = bars + 0;     // Q chunk landed                                   (TMA -> MMA)
  uint64_t* k_full = bars + 1;     // K chunk landed
  uint64_t* v_full = bars + 2;     // V chunk landed
  uint64_t* q_free = bars + 3;     // Z and Q S of the chunk complete                   (MMA -> TMA)
  uint64_t* k_free = bars + 4;     // state update of the chunk complete: K free        (MMA -> TMA)
  uint64_t* z_full = bars + 5;     // Z complete                                        (MMA -> element-wise)
  uint64_t* w_full = bars + 6;     // W written over Z and the carried term scaled       (element-wise -> MMA), 128 arrivals
  uint64_t* acc_done = bars + 7;   // ACC of the chunk complete                         (MMA -> element-wise)
  uint64_t* acc_free = bars + 8;   // ACC read into registers                           (element-wise -> MMA), 128 arrivals
  uint64_t* u_done = bars + 9;     // state update of the chunk complete                (MMA -> element-wise)
  uint64_t* s_ready = bars + 10;   // decayed state in TMEM and its 16-bit copy in smem (element-wise -> MMA), 128 arrivals
  uint64_t* y_done = bars + 11;    // Q S complete                                      (MMA -> element-wise)
  uint64_t* k_scaled = bars + 12;  // rows of the K tile scaled in place                (element-wise -> MMA), 128 arrivals
  uint64_t* v_free = bars + 13;    // the chunk's output, staged in the V tile, has left it (row warps -> TMA), 4 arrivals
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 14);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int n_off = blockIdx.x * DVC;
  const int nchunk_all = (p.L + 127) / 128;
  const int seg_id = blockIdx.z;
  const int c_begin = seg_id * p.seg;                         // first chunk of this CTA's segment
  const int nchunk = min(nchunk_all - c_begin, p.seg);        // chunks this CTA walks (local index c below)
  const bool init = seg_id > 0;                               // starts from the state the earlier segments leave behind
  const uint32_t sb = init ? 1u : 0u;                         // that state is one more arrival on s_ready / y_done

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(k_full, 1);
    mbar_init(v_full, 1);
    mbar_init(q_free, 1);
    mbar_init(k_free, 1);
    mbar_init(v_free, 4);
    mbar_init(z_full, 1);
    mbar_init(w_full, 128);
    mbar_init(acc_done, 1);
    mbar_init(acc_free, 128);
    mbar_init(u_done, 1);
    mbar_init(s_ready, 128);
    mbar_init(y_done, 1);
    mbar_init(k_scaled, 128);
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_base_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmO);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const uint32_t tZ = tmem_base;
  const uint32_t tACC = tmem_base + 128;
  const uint32_t tS = tmem_base + 256;  // half h at tS + 128 * h

  if (warp == 9) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      bool ok = true;
      int nq = 0, nk = 0, nkv = 0;  // chunks whose Q / K / V loads have been issued
      for (int c = 0; c < nchunk && ok; ++c) {
        if (c > 0) ok = mbar_wait(q_free, (c - 1) & 1, ab, kRcQFree);
        if (!ok) break;
        AB200_CTR(1, c, 4);
        mbar_expect_tx(q_full, Cfg::QK_BYTES);
#pragma unroll
        for (int b = 0; b < KB; ++b) tma_load_3d(sQ + b * BOX, &tmQ, q_full, b * 64, (c_begin + c) * 128, bh);
        ++nq;
        if (c > 0) ok = mbar_wait(k_free, (c - 1) & 1, ab, kRcKVFree);
        if (!ok) break;
        AB200_CTR(1, c, 5);
        mbar_expect_tx(k_full, Cfg::QK_BYTES);
#pragma unroll
        for (int b = 0; b < KB; ++b) tma_load_3d(sK + b * BOX, &tmK, k_full, b * 64, (c_begin + c) * 128, bh);
        ++nk;
        if (c > 0) ok = mbar_wait(v_free, (c - 1) & 1, ab, kRcKVFree);
        if (!ok) break;
        AB200_CTR(1, c, 6);
        mbar_expect_tx(v_full, Cfg::V_BYTES);
#pragma unroll
        for (int b = 0; b < VB; ++b) tma_load_3d(sV + b * BOX, &tmV, v_full, n_off + b * 64, (c_begin + c) * 128, bh);
        ++nkv;
        if (c + 1 < nchunk) {
          // the buffers are single (shared memory is full at dqk = 256), so the next chunk's loads start only when this
          // chunk's MMAs have released them: ask the L2 for those tiles now, so that they come from L2 rather than HBM
#pragma unroll
          for (int b = 0; b < KB; ++b) {
            tma_prefetch_3d(&tmQ, b * 64, (c_begin + c + 1) * 128, bh);
            tma_prefetch_3d(&tmK, b * 64, (c_begin + c + 1) * 128, bh);
          }
#pragma unroll
          for (int b = 0; b < VB; ++b) tma_prefetch_3d(&tmV, n_off + b * 64, (c_begin + c + 1) * 128, bh);
        }
      }
      if (!ok) {
        // abort path: let the copies already issued land before this CTA's shared memory is released
        if (nq > 0) mbar_wait_drain(q_full, (nq - 1) & 1, 2000000ull);
        if (nk > 0) mbar_wait_drain(k_full, (nk - 1) & 1, 2000000ull);
        if (nkv > 0) mbar_wait_drain(v_full, (nkv - 1) & 1, 2000000ull);
      }
    }
  } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer (converged warp, one elected lane)
    constexpr uint32_t idesc_z = umma_idesc(128, 128, BF16, false, false);   // Q K^T: both K-major
    constexpr uint32_t idesc_y = umma_idesc(128, DVC, BF16, false, true);    // Q S, W V: B MN-major
    constexpr uint32_t idesc_u = umma_idesc(128, DVC, BF16, true, true);     // K^T V: A and B MN-major
    const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV), sb_addr = smem_u32(sSb);
    bool ok = true;
    for (int c = 0; c < nchunk && ok; ++c) {
      const uint32_t ph = c & 1;
      ok = mbar_wait_warp(q_full, ph, ab, kRcQ);
      if (ok) ok = mbar_wait_warp(k_full, ph, ab, kRcK);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) AB200_CTR(1, c, 0);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < DQK / 16; ++ks) {
          const uint32_t off = (ks >> 2) * BOX + (ks & 3) * 32;
          umma_ss(tZ, umma_smem_desc(q_addr + off, 16, 1024), umma_smem_desc(k_addr + off, 16, 1024), idesc_z, ks > 0 ? 1u : 0u);
        }
        tc_commit(z_full);
      }
      __syncwarp();
      const bool carried = c > 0 || init;
      if (carried) {
        // the carried state: its 16-bit copy is in shared memory and ACC of the previous chunk has been read
        ok = mbar_wait_warp(s_ready, (c - 1 + sb) & 1, ab, kRcState);
        if (ok && c > 0) ok = mbar_wait_warp(acc_free, (c - 1) & 1, ab, kRcAccFree);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0) AB200_CTR(1, c, 1);
        if (elect_one()) {
#pragma unroll
          for (int ks = 0; ks < DQK / 16; ++ks) {
            const uint32_t qoff = (ks >> 2) * BOX + (ks & 3) * 32;
            const uint32_t soff = (ks >> 3) * Cfg::SB_HALF_BYTES + (ks & 7) * 2048;
            umma_ss(tACC, umma_smem_desc(q_addr + qoff, 16, 1024), umma_smem_desc(sb_addr + soff, BOX, 1024), idesc_y,
                    ks > 0 ? 1u : 0u);
          }
          tc_commit(y_done);
        }
        __syncwarp();
      }
      if (elect_one()) tc_commit(q_free);  // Z and Q S are the only readers of the Q chunk
      __syncwarp();
      // state update as soon as the rows of the K tile carry gamma^(127-j): S_h (already multiplied by g) += K_c[:, half h]^T V_c
      ok = mbar_wait_warp(v_full, ph, ab, kRcV);
      if (ok) ok = mbar_wait_warp(k_scaled, ph, ab, kRcKScaled);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) AB200_CTR(1, c, 2);
      if (elect_one()) {
#pragma unroll
        for (int h = 0; h < NH; ++h) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ss(tS + h * 128, umma_smem_desc(k_addr + (2 * h) * BOX + ks * 2048, BOX, 1024),
                    umma_smem_desc(v_addr + ks * 2048, BOX, 1024), idesc_u, (carried || ks > 0) ? 1u : 0u);
        }
        tc_commit(u_done);
        tc_commit(k_free);  // the next chunk's K tile loads under this chunk's W V
      }
      __syncwarp();
      ok = mbar_wait_warp(w_full, ph, ab, kRcW);
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) AB200_CTR(1, c, 3);
      if (elect_one()) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(tACC, tZ + ks * 8, umma_smem_desc(v_addr + ks * 2048, BOX, 1024), idesc_y, (carried || ks > 0) ? 1u : 0u);
        tc_commit(acc_done);
      }
      __syncwarp();
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ state warpgroup (warps 4-7): rows of the K tile
    // and rows of the state. Thread t owns TMEM lane t = row t of each state half.
    const int wq = warp - 4;
    const int tid = threadIdx.x - 128;
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32);
    const float lg = log2f(p.decay[bh % p.H]);
    const float g128 = exp2f(128.0f * lg);
    const uint64_t g2 = f2_pack(g128, g128);
    // 32 columns of row `tid` of state half hh, fp32 in rr: 16-bit copy into shared memory (operand of the next Q S; four
    // 16-byte groups of the row's 128-byte line in box c0 / 64, 128-byte swizzle), and g * S into tensor memory, where
    // the next chunk's K^T V is added
    auto put_state = [&](int hh, int c0, uint32_t (&rr)[32]) {
      uint8_t* box = sSb + hh * Cfg::SB_HALF_BYTES + tid * 128 + (c0 >> 6) * BOX;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint4 v;
        v.x = pack2<BF16>(__uint_as_float(rr[q4 * 8 + 0]), __uint_as_float(rr[q4 * 8 + 1]));
        v.y = pack2<BF16>(__uint_as_float(rr[q4 * 8 + 2]), __uint_as_float(rr[q4 * 8 + 3]));
        v.z = pack2<BF16>(__uint_as_float(rr[q4 * 8 + 4]), __uint_as_float(rr[q4 * 8 + 5]));
        v.w = pack2<BF16>(__uint_as_float(rr[q4 * 8 + 6]), __uint_as_float(rr[q4 * 8 + 7]));
        const int chunk16 = ((c0 & 63) >> 3) + q4;
        *reinterpret_cast<uint4*>(box + ((chunk16 ^ (tid & 7)) << 4)) = v;
      }
#pragma unroll
      for (int i = 0; i < 32; i += 2) {
        float x0, x1;
        f2_unpack(fmul2(f2_pack(__uint_as_float(rr[i]), __uint_as_float(rr[i + 1])), g2), x0, x1);
        rr[i] = __float_as_uint(x0);
        rr[i + 1] = __float_as_uint(x1);
      }
      tmem_st32(tmem_addr(tS + hh * 128, lane_base, 0) + c0, rr);
    };
    bool ok = true;
    if (init) {
      // ---- the state the earlier segments leave behind: T_g' carried over the segments between g' and this one
      const float* ws_tile = p.ws + (static_cast<size_t>(bh) * gridDim.x + blockIdx.x) * (gridDim.z - 1) * (DQK * DVC);
#pragma unroll 1
      for (int hh = 0; hh < NH; ++hh) {
#pragma unroll 1
        for (int c0 = 0; c0 < DVC; c0 += 32) {
          float acc[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = 0.f;
          for (int gp = seg_id - 1; gp >= 0; --gp) {
            const float f = exp2f(128.0f * p.seg * (seg_id - 1 - gp) * lg);
            if (f == 0.f) break;  // the same for every thread; earlier segments weigh even less
            const float* src = ws_tile + (static_cast<size_t>(gp) * NH + hh) * (DVC * 128) + c0 * 128 + tid;
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = fmaf(f, src[i * 128], acc[i]);
          }
          uint32_t rr[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) rr[i] = __float_as_uint(acc[i]);
          put_state(hh, c0, rr);
        }
      }
      tc_wait_st();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(s_ready);
    }
    for (int c = 0; c < nchunk && ok; ++c) {
      const uint32_t ph = c & 1;
      ok = mbar_wait_warp(z_full, ph, ab, kRcZ);
      if (ok) ok = mbar_wait_warp(k_full, ph, ab, kRcK);  // long complete; makes the TMA's writes visible to this thread
      if (!ok) break;
      // ---- Q K^T has read the plain K tile: scale its rows in place for the state update. A row takes one factor, so
      //      the work is shared by address, not by row: the 32 lanes of a warp cover four consecutive 128-byte lines at a
      //      time (lane l: line l / 8, 16-byte group l % 8), which is free of bank conflicts; a thread per row would put
      //      all lanes of a warp on the same banks.
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int krow_idx = wq * 32 + it * 4 + (lane >> 3);
        const float kf = exp2f((127 - krow_idx) * lg);  // gamma^(127-j)
        const uint32_t kr2 = pack2<BF16>(kf, kf);       // one packed 16-bit product per pair (a factor rounded to 16
                                                        // bits costs what the rounding of the product costs)
#pragma unroll
        for (int b = 0; b < KB; ++b) {
          uint4* ptr = reinterpret_cast<uint4*>(sK + b * BOX + krow_idx * 128 + (lane & 7) * 16);
          uint4 u = *ptr;
          *ptr = make_uint4(mul2_16<BF16>(u.x, kr2), mul2_16<BF16>(u.y, kr2), mul2_16<BF16>(u.z, kr2), mul2_16<BF16>(u.w, kr2));
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(k_scaled);
      if (tid == 0) AB200_CTR(0, c, 5);
      // ---- carried state for the next chunk: 16-bit copy of S into shared memory, S <- g S in tensor memory. The commit
      //      behind u_done follows the chunk's Q S in the issuing thread, so the copy that Q S read is free as well.
      if (c + 1 < nchunk) {
        ok = mbar_wait_warp(u_done, ph, ab, kRcU);
        if (!ok) break;
        tc_fence_after();
        if (tid == 0) AB200_CTR(0, c, 6);
        // blocks of 32 columns, two in flight: the load of the next block runs under the work on this one
        constexpr int NBLK = NH * (DVC / 32);
        auto blk_addr = [&](int blk) { return tmem_addr(tS + (blk / (DVC / 32)) * 128, lane_base, 0) + (blk % (DVC / 32)) * 32; };
        uint32_t ra[32], rb[32];
        tmem_ld32(blk_addr(0), ra);
#pragma unroll 1
        for (int blk = 0; blk < NBLK; blk += 2) {
          tc_wait_ld();
          tmem_ld32(blk_addr(blk + 1), rb);
          put_state(blk / (DVC / 32), (blk % (DVC / 32)) * 32, ra);
          tc_wait_ld();
          if (blk + 2 < NBLK) tmem_ld32(blk_addr(blk + 2), ra);
          put_state((blk + 1) / (DVC / 32), ((blk + 1) % (DVC / 32)) * 32, rb);
        }
        tc_wait_st();
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(s_ready);
        if (tid == 0) AB200_CTR(0, c, 7);
      }
    }
  } else {
    // ------------------------------------------------------------------ row warpgroup (warps 0-3): thread t owns TMEM
    // lane t = row t of the chunk in Z and ACC
    const int tid = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32);
    const float lg = log2f(p.decay[bh % p.H]);
    const float row_decay = exp2f(tid * lg);                 // gamma^i, row factor of W (columns bring gamma^-j)
    const float carry = exp2f((tid + 1) * lg);               // gamma^(i+1): the carried state seen from row i
    const uint64_t carry2 = f2_pack(carry, carry);
    const uint64_t sc2 = f2_pack(p.scale, p.scale);
    const uint32_t tz = tmem_addr(tZ, lane_base, 0);
    const uint32_t ta = tmem_addr(tACC, lane_base, 0);
    bool ok = true;
    for (int c = 0; c < nchunk && ok; ++c) {
      const uint32_t ph = c & 1;
      // ---- W = Z .* gamma^(i-j), keys after the row's own position removed (the forward flavour of the chain kernels'
      //      element-wise step: row factor gamma^i, running column factor gamma^-j, triangular predicate)
      ok = mbar_wait_warp(z_full, ph, ab, kRcZ);
      if (!ok) break;
      tc_fence_after();
      if (tid == 0) AB200_CTR(0, c, 0);
      {
        float unused_sum = 0.f;
        chain_ew_decay2<kChainFwd, BF16, 0, false>(tz, row_decay, lg, 0.f, 0.f, true, tid, unused_sum);
        chain_ew_decay2<kChainFwd, BF16, 2, false>(tz, row_decay, lg, 0.f, 0.f, true, tid, unused_sum);
      }
      if (tid == 0) AB200_CTR(0, c, 1);
      // ---- the carried term Q S, now in ACC, seen from row i: times gamma^(i+1)
      if (c > 0 || init) {
        ok = mbar_wait_warp(y_done, (c - 1 + sb) & 1, ab, kRcY);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < DVC; c0 += 32) {
          uint32_t rr[32];
          tmem_ld32(ta + c0, rr);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0, x1;
            f2_unpack(fmul2(f2_pack(__uint_as_float(rr[i]), __uint_as_float(rr[i + 1])), carry2), x0, x1);
            rr[i] = __float_as_uint(x0);
            rr[i + 1] = __float_as_uint(x1);
          }
          tmem_st32(ta + c0, rr);
        }
      }
      tc_wait_st();
      tc_fence_before();
      mbar_arrive(w_full);
      if (tid == 0) AB200_CTR(0, c, 2);
      // ---- O_c = scale * ACC
      ok = mbar_wait_warp(acc_done, ph, ab, kRcAcc);
      if (!ok) break;
      tc_fence_after();
      if (tid == 0) AB200_CTR(0, c, 3);
      {
        // W V was the last reader of the V tile, which has the size and the layout of this CTA's piece of the output: the
        // rows go there (16-bit, 128-byte swizzle) and leave through TMA stores, one per warp and 64-column box (32 rows
        // each, so no warp waits for another); rows past the end of the sequence are clipped by the store
        uint8_t* stage = sV + tid * 128;
#pragma unroll
        for (int c0 = 0; c0 < DVC; c0 += 32) {
          uint32_t rr[32];
          tmem_ld32(ta + c0, rr);
          tc_wait_ld();
          if (c0 + 32 >= DVC) {
            tc_fence_before();
            mbar_arrive(acc_free);
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint32_t v[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float x0, x1;
              f2_unpack(fmul2(f2_pack(__uint_as_float(rr[q4 * 8 + 2 * e]), __uint_as_float(rr[q4 * 8 + 2 * e + 1])), sc2), x0, x1);
              v[e] = pack2<BF16>(x0, x1);
            }
            const int chunk16 = ((c0 & 63) >> 3) + q4;
            *reinterpret_cast<uint4*>(stage + (c0 >> 6) * BOX + ((chunk16 ^ (tid & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          const int row0 = (c_begin + c) * 128 + warp * 32;
          if (row0 < p.L) {
#pragma unroll
            for (int b = 0; b < VB; ++b) tma_store_3d(&tmO, sV + b * BOX + warp * 32 * 128, n_off + b * 64, row0, bh);
            tma_store_commit();
            tma_store_wait_read0();
          }
          mbar_arrive(v_free);
        }
      }
      if (tid == 0) AB200_CTR(0, c, 4);
    }
    if (lane == 0) tma_store_wait0();  // all output written before the CTA exits
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// State of one segment taken alone: T = sum over the segment's chunks c and positions j of
// gamma^(127 - j + 128 (last - c)) k_j v_j^T, which is what the walk in order would add to its state over these
// chunks. The whole decay sits on the rows of K (scaled in place in shared memory, like the state update of the kernel
// above), so the accumulator in tensor memory is touched by nothing but the MMAs: a row whose factor underflows in
// 16 bits is a contribution that small. Grid (dv / DVC, BH, segments - 1); K and V tiles in a ring of two. Warps 0-3
// scale the K rows, warp 4 issues the MMAs, warp 5 lane 0 is the TMA producer. Output: fp32, [state half][column][row]
// per CTA, so that both this kernel's stores and the consumer's loads (a thread per state row) are coalesced.
template <class Cfg>
struct RetChunkStateLayout {
  static constexpr int STAGE_BYTES = Cfg::QK_BYTES + Cfg::V_BYTES;
  static constexpr int SMEM_TILES = 2 * STAGE_BYTES;
  static constexpr int SMEM_BYTES = 1024 + SMEM_TILES + 512;
  static constexpr int TMEM_COLS = 256;
  static constexpr int NTHREADS = 192;
  static_assert(SMEM_BYTES <= 232448, "shared memory");
  static_assert(Cfg::NH * 128 <= TMEM_COLS, "tensor memory");
};

template <class Cfg>
__global__ void __launch_bounds__(RetChunkStateLayout<Cfg>::NTHREADS, 1)
ret_chunk_state_sm100_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                             const RetChunkParams p) {
  using Lay = RetChunkStateLayout<Cfg>;
  constexpr int DQK = Cfg::DQK, DVC = Cfg::DVC, NH = Cfg::NH, KB = Cfg::KB, VB = Cfg::VB, BOX = Cfg::BOX_BYTES;
  constexpr bool BF16 = Cfg::BF16;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Lay::SMEM_TILES);
  uint64_t* kv_full = bars + 0;    // [2] K and V of a chunk landed                    (TMA -> element-wise, MMA)
  uint64_t* kv_empty = bars + 2;   // [2] the chunk's MMAs complete                     (MMA -> TMA)
  uint64_t* k_scaled = bars + 4;   // [2] rows of the K tile scaled in place            (element-wise -> MMA), 128 arrivals
  uint64_t* s_done = bars + 6;     // every MMA of the segment complete                 (MMA -> element-wise)
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(bars + 7);
  CtaAbort* ab = reinterpret_cast<CtaAbort*>(tmem_base_slot + 1);

  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const int lane = threadIdx.x & 31;
  const int bh = blockIdx.y;
  const int n_off = blockIdx.x * DVC;
  const int c_begin = blockIdx.z * p.seg;
  const int nchunk = p.seg;  // every segment but the last is whole

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
      mbar_init(k_scaled + s, 128);
    }
    mbar_init(s_done, 1);
    ab->flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_base_slot, Lay::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 5 && lane == 0) {
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 5) {
    if (lane == 0) {
      bool ok = true;
      int nload = 0;
      for (int c = 0; c < nchunk && ok; ++c) {
        const int s = c & 1;
        if (c >= 2) ok = mbar_wait(kv_empty + s, ((c >> 1) - 1) & 1, ab, kRsEmpty);
        if (!ok) break;
        uint8_t* sK = smem + s * Lay::STAGE_BYTES;
        uint8_t* sV = sK + Cfg::QK_BYTES;
        mbar_expect_tx(kv_full + s, Lay::STAGE_BYTES);
#pragma unroll
        for (int b = 0; b < KB; ++b) tma_load_3d(sK + b * BOX, &tmK, kv_full + s, b * 64, (c_begin + c) * 128, bh);
#pragma unroll
        for (int b = 0; b < VB; ++b) tma_load_3d(sV + b * BOX, &tmV, kv_full + s, n_off + b * 64, (c_begin + c) * 128, bh);
        ++nload;
      }
      if (!ok) {
        // abort path: let the copies already issued land before this CTA's shared memory is released
        if (nload > 0) mbar_wait_drain(kv_full + ((nload - 1) & 1), ((nload - 1) >> 1) & 1, 2000000ull);
        if (nload > 1) mbar_wait_drain(kv_full + ((nload - 2) & 1), ((nload - 2) >> 1) & 1, 2000000ull);
      }
    }
  } else if (warp == 4) {
    constexpr uint32_t idesc_u = umma_idesc(128, DVC, BF16, true, true);  // K^T V: A and B MN-major
    bool ok = true;
    for (int c = 0; c < nchunk && ok; ++c) {
      const int s = c & 1;
      const uint32_t ph = (c >> 1) & 1;
      ok = mbar_wait_warp(kv_full + s, ph, ab, kRsFull);
      if (ok) ok = mbar_wait_warp(k_scaled + s, ph, ab, kRsScaled);
      if (!ok) break;
      tc_fence_after();
      if (elect_one()) {
        const uint32_t k_addr = smem_u32(smem + s * Lay::STAGE_BYTES), v_addr = k_addr + Cfg::QK_BYTES;
#pragma unroll
        for (int h = 0; h < NH; ++h) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ss(tmem_base + h * 128, umma_smem_desc(k_addr + (2 * h) * BOX + ks * 2048, BOX, 1024),
                    umma_smem_desc(v_addr + ks * 2048, BOX, 1024), idesc_u, (c > 0 || ks > 0) ? 1u : 0u);
        }
        tc_commit(kv_empty + s);
        if (c + 1 == nchunk) tc_commit(s_done);
      }
      __syncwarp();
    }
  } else {
    const int tid = threadIdx.x;
    const uint32_t lane_base = static_cast<uint32_t>(warp * 32);
    const float lg = log2f(p.decay[bh % p.H]);
    bool ok = true;
    for (int c = 0; c < nchunk && ok; ++c) {
      const int s = c & 1;
      ok = mbar_wait_warp(kv_full + s, (c >> 1) & 1, ab, kRsFull);
      if (!ok) break;
      uint8_t* sK = smem + s * Lay::STAGE_BYTES;
      const int later = 128 * (nchunk - 1 - c);  // positions of the segment after this chunk
      // shared by address (lane l: line l / 8, 16-byte group l % 8), free of bank conflicts
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int krow_idx = warp * 32 + it * 4 + (lane >> 3);
        const float kf = exp2f((127 - krow_idx + later) * lg);
        const uint32_t kr2 = pack2<BF16>(kf, kf);
#pragma unroll
        for (int b = 0; b < KB; ++b) {
          uint4* ptr = reinterpret_cast<uint4*>(sK + b * BOX + krow_idx * 128 + (lane & 7) * 16);
          uint4 u = *ptr;
          *ptr = make_uint4(mul2_16<BF16>(u.x, kr2), mul2_16<BF16>(u.y, kr2), mul2_16<BF16>(u.z, kr2), mul2_16<BF16>(u.w, kr2));
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(k_scaled + s);
    }
    if (ok) ok = mbar_wait_warp(s_done, 0, ab, kRsDone);
    if (ok) {
      tc_fence_after();
      float* dst = p.ws + ((static_cast<size_t>(bh) * gridDim.x + blockIdx.x) * gridDim.z + blockIdx.z) * (DQK * DVC) + tid;
#pragma unroll 1
      for (int hh = 0; hh < NH; ++hh) {
#pragma unroll 1
        for (int c0 = 0; c0 < DVC; c0 += 32) {
          uint32_t rr[32];
          tmem_ld32(tmem_addr(tmem_base + hh * 128, lane_base, 0) + c0, rr);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) dst[(hh * DVC + c0 + i) * 128] = __uint_as_float(rr[i]);
        }
      }
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Lay::TMEM_COLS);
  }
}

}  // namespace ab200
