// Declarations shared by the two-GEMM chain kernels (single CTA: chain_sm100.cuh, CTA pair:
// chain_pair_sm100.cuh): work-item description, kernel parameters and the element-wise step
//     W = Z .* mask .* scale (./ r)
// that runs between the two GEMMs on one 128 x 128 block held in tensor memory.
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
  const uint16_t* mask_t;  // RowK flavours only: transposed copy [H, Lkv, Lq] of the mask in scratch memory, or nullptr
  const float* decay;    // per-head gamma [H] or nullptr (exactly one of mask / decay is set)
  int H, Lq, Lkv;
  float scale;
  int skip_upper;        // 1: blocks strictly above the diagonal are all zero and are skipped
  // work list of the persistent grid: item w = (bh * ny + chunk) * nrb + row-block index
  int nrb;               // 128-row blocks on the row side
  int ny;                // column chunks of the output (n2_total / N2)
  int total_items;       // nrb * ny * BH
};

// One unit of work of the persistent chain kernel: a 128-row tile x one output-column chunk of one slice.
struct ChainItem {
  int bh, n_off, row0, t_start, n_iter;
};

// Optional event trace (compile with -DAB200_TRACE), see fa_fwd_sm100.cuh: CTA (0,0,0) only.
#ifdef AB200_TRACE
constexpr int kChainTraceIters = 48;
__device__ long long g_chain_trace[2][kChainTraceIters][8];
#define AB200_CTR(who, j, ev)                                                                            \
  do {                                                                                                   \
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && (j) < kChainTraceIters) g_chain_trace[who][j][ev] = clock64(); \
  } while (0)
#else
#define AB200_CTR(who, j, ev) do {} while (0)
#endif

// Tags of the bounded waits (reported in the device status detail word)
enum ChainTag : int {
  kCtR = 11, kCtSlotFull = 12, kCtSlotEmpty = 13, kCtZFull = 14, kCtWFull = 15, kCtAccDone = 16, kCtAccFree = 17, kCtRFree = 18, kCtZFree = 19
};

// The forward keeps W = S~ UNNORMALISED in 16 bits (the division by r happens once, in the epilogue), whereas the
// reference divides by the running r before the fp16 cast (csrc/kernels/retnet/regfuse/regfuse.h:306-316) and can
// never leave the fp16 range. cvt.rn.satfinite clamps |S~| > 65504 silently, which would make the output wrong, so a
// clamp is detected and reported (status 2, read by the host like a timeout). No element can exceed 65504 unless the
// running sum of |W| over the thread's columns does, so the common case costs one comparison per 32 columns; only
// then are the packed values inspected.
__device__ __forceinline__ void chain_check_saturation(float abs_sum_so_far, const uint32_t (&pk)[16]) {
  if (abs_sum_so_far > 65504.0f) {
    bool sat = false;
#pragma unroll
    for (int i = 0; i < 16; ++i) sat |= half2_has_maxnorm(pk[i]);
    if (sat) report_saturation();
  }
}

// Element-wise step of one block, W = Z .* mask .* scale (./ r), for the thread that owns TMEM lane (row) `tz >> 16`:
// it reads fp32 values of its row of Z at `tz`, applies the row factor and the mask (decay factors built in
// registers, or a general 16-bit mask tensor) and writes packed 16-bit pairs of W over the first columns of the same
// buffer; the forward accumulates sum |W|. Every flavour handles two 32-column chunks (QD0, QD0 + 1) per call. With
// SPLITW two threads share a row (chunks 0-1 and 2-3) and each keeps its 32 packed W columns inside its own half of
// the buffer: W of chunks 0-1 at columns [0,32), of chunks 2-3 at [64,96); otherwise W sits at columns [0,64).
//
// Decay flavours (no mask tensor), written for instruction count and without shared-memory reads. Measured alone on
// one SM, cycles per 128 x 128 block with two threads per row: 980 for a straightforward loop that reads a
// column-factor table from shared memory; 534 for this version; and with SS MMAs streaming their operands from
// shared memory on the same SM the table version (one broadcast read per 4 columns) took 2611 cycles against 550
// here: the tensor core saturates the shared-memory bandwidth and starves LDS.
//   * Fwd / RowQ: the column factor gamma^(-c) is a running product, two columns per packed multiply,
//     restarted from an exact value at every chunk (32 steps of fp32 rounding at most);
//   * RowK: the column factor gamma^c / r[c] of column (chunk, lane) sits in a register of that lane
//     (colf0 / colf1 for the two chunks) and travels by warp shuffle;
//   * both TMEM loads are issued before the first wait; the row sum uses four independent accumulators.
// rowf is the per-row factor; lg = log2(gamma).
template <int MODE, bool BF16, int QD0, bool SPLITW>
__device__ __forceinline__ void chain_ew_decay2(uint32_t tz, float rowf, float lg, float colf0, float colf1, bool straddle,
                                                int dlim, float& rsum) {
  uint32_t zr[2][32];
  tmem_ld32(tz + QD0 * 32, zr[0]);
  tmem_ld32(tz + (QD0 + 1) * 32, zr[1]);
  const uint64_t rf2 = f2_pack(rowf, rowf);
  const float ginv = exp2f(-lg);
  const uint64_t step2 = f2_pack(ginv * ginv, ginv * ginv);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  tc_wait_ld();
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t pk[16];
    uint64_t g = 0;
    if (MODE != kChainRowK) {
      const float f0 = rowf * exp2f(-((QD0 + q) * 32) * lg);
      g = f2_pack(f0, f0 * ginv);
    }
    const float colf = q == 0 ? colf0 : colf1;
#pragma unroll
    for (int c4 = 0; c4 < 8; ++c4) {
      uint64_t a = f2_pack(__uint_as_float(zr[q][4 * c4]), __uint_as_float(zr[q][4 * c4 + 1]));
      uint64_t b = f2_pack(__uint_as_float(zr[q][4 * c4 + 2]), __uint_as_float(zr[q][4 * c4 + 3]));
      if (MODE == kChainRowK) {
        const float fa = __shfl_sync(0xffffffffu, colf, 4 * c4), fb = __shfl_sync(0xffffffffu, colf, 4 * c4 + 1);
        const float fc = __shfl_sync(0xffffffffu, colf, 4 * c4 + 2), fd = __shfl_sync(0xffffffffu, colf, 4 * c4 + 3);
        a = fmul2(fmul2(a, rf2), f2_pack(fa, fb));
        b = fmul2(fmul2(b, rf2), f2_pack(fc, fd));
      } else {
        a = fmul2(a, g);
        g = fmul2(g, step2);
        b = fmul2(b, g);
        g = fmul2(g, step2);
      }
      float w0, w1, w2, w3;
      f2_unpack(a, w0, w1);
      f2_unpack(b, w2, w3);
      if (straddle) {  // warp-uniform: only blocks on the diagonal pay for the triangular predicate
        const int cc = (QD0 + q) * 32 + 4 * c4;
        if (MODE == kChainRowK) {
          if (cc < dlim) w0 = 0.f;
          if (cc + 1 < dlim) w1 = 0.f;
          if (cc + 2 < dlim) w2 = 0.f;
          if (cc + 3 < dlim) w3 = 0.f;
        } else {
          if (cc > dlim) w0 = 0.f;
          if (cc + 1 > dlim) w1 = 0.f;
          if (cc + 2 > dlim) w2 = 0.f;
          if (cc + 3 > dlim) w3 = 0.f;
        }
      }
      if (MODE == kChainFwd) {
        s0 += fabsf(w0);
        s1 += fabsf(w1);
        s2 += fabsf(w2);
        s3 += fabsf(w3);
      }
      pk[2 * c4] = pack2<BF16>(w0, w1);
      pk[2 * c4 + 1] = pack2<BF16>(w2, w3);
    }
    if constexpr (MODE == kChainFwd && !BF16) chain_check_saturation((s0 + s1) + (s2 + s3), pk);
    tmem_st16(tz + (SPLITW ? (QD0 >> 1) * 64 + q * 16 : (QD0 + q) * 16), pk);
  }
  if (MODE == kChainFwd) rsum += (s0 + s1) + (s2 + s3);
}

// Column factor of the RowK flavours for the decay mask: gamma^c / r[query col0 + c], for the lane's column of
// 32-column chunk `chunk` (0 for queries past the end).
__device__ __forceinline__ float chain_rowk_colf(const ChainParams& p, int bh, int col0, int chunk, int lane, float lg) {
  const int c = chunk * 32 + lane;
  const int qi = col0 + c;
  const float f = (qi < p.Lq) ? 1.0f / p.r_in[static_cast<size_t>(bh) * p.Lq + qi] : 0.f;
  return f * exp2f(c * lg);
}

// ---- mask-tensor flavours, two 32-column chunks (QD0, QD0 + 1) per thread
// The mask values a thread needs for one block are fetched BEFORE it waits for Z (their latency then runs under
// GEMM1) and kept packed, two 16-bit values per register: mk[i] = columns (2i, 2i+1) of the thread's 64 columns.
//   Fwd / RowQ: row `grow` of M[h], columns col0 + 32 QD0 ... : eight 16-byte loads.
template <int MODE, int QD0>
__device__ __forceinline__ void chain_mask_prefetch(const ChainParams& p, int h, int grow, int col0, uint32_t (&mk)[32]) {
  static_assert(MODE != kChainRowK, "row reads only");
  const uint16_t* mp = p.mask + (static_cast<size_t>(h) * p.Lq + grow) * p.Lkv + col0 + QD0 * 32;
#pragma unroll
  for (int v8 = 0; v8 < 8; ++v8) {
    uint4 u = make_uint4(0, 0, 0, 0);
    if (grow < p.Lq && col0 + QD0 * 32 + v8 * 8 < p.Lkv) u = __ldg(reinterpret_cast<const uint4*>(mp) + v8);
    mk[4 * v8 + 0] = u.x;
    mk[4 * v8 + 1] = u.y;
    mk[4 * v8 + 2] = u.z;
    mk[4 * v8 + 3] = u.w;
  }
}

//   RowK with a transposed copy of the mask (mask_t[h][key][query], made once per backward call in scratch memory by
//   mask_transpose_kernel): the thread's column of the mask is a row of the copy, read like the Fwd / RowQ rows.
template <int QD0>
__device__ __forceinline__ void chain_mask_prefetch_t(const ChainParams& p, int h, int key, int col0, uint32_t (&mk)[32]) {
  const uint16_t* mp = p.mask_t + (static_cast<size_t>(h) * p.Lkv + key) * p.Lq + col0 + QD0 * 32;
#pragma unroll
  for (int v8 = 0; v8 < 8; ++v8) {
    uint4 u = make_uint4(0, 0, 0, 0);
    if (key < p.Lkv && col0 + QD0 * 32 + v8 * 8 < p.Lq) u = __ldg(reinterpret_cast<const uint4*>(mp) + v8);
    mk[4 * v8 + 0] = u.x;
    mk[4 * v8 + 1] = u.y;
    mk[4 * v8 + 2] = u.z;
    mk[4 * v8 + 3] = u.w;
  }
}

// out[h][j][i] = in[h][i][j] for a 16-bit tensor in [H, rows, cols]: 32 x 32 tiles through shared memory (padded rows,
// no bank conflicts), coalesced on both sides. grid = (ceil(cols / 32), ceil(rows / 32), H), block = (32, 8).
__global__ void mask_transpose_kernel(const uint16_t* __restrict__ in, uint16_t* __restrict__ out, int rows, int cols) {
  __shared__ uint16_t tile[32][34];
  const size_t plane = static_cast<size_t>(rows) * cols;
  const uint16_t* src = in + blockIdx.z * plane;
  uint16_t* dst = out + blockIdx.z * plane;
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
#pragma unroll
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    tile[i][threadIdx.x] = (r < rows && c < cols) ? src[static_cast<size_t>(r) * cols + c] : uint16_t(0);
  }
  __syncthreads();
#pragma unroll
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int c = c0 + i, r = r0 + threadIdx.x;  // out row = in column
    if (c < cols && r < rows) dst[static_cast<size_t>(c) * rows + r] = tile[threadIdx.x][i];
  }
}

// RowK flavours: thread (lane L of its warp) owns key grow0 + L and needs M[h][query][key] for the 64 queries of its
// two chunks, i.e. a COLUMN of the mask. Reading it with 64 two-byte loads per thread and block cost 0.9 ms of the
// 1.55 ms backward at config 4 (measured by replacing the loads with a constant). Here the warp reads its
// 32-query x 32-key tile of every chunk by rows with four 16-byte loads per lane (lane l: key group l / 8, rows
// 8 i + l % 8) and transposes it in registers: every group of 8 lanes holds an 8 x 8 block of 16-bit values, one row
// per lane, and exchanges halves three times (lane distance 4, 2, 1; shuffles and byte permutes) until lane j holds
// column j, packed as (row 2n, row 2n+1) pairs, which is the layout chain_ew_mask2 wants.
__device__ __forceinline__ void chain_transpose8x8_b16(uint32_t (&r)[4], int lane) {
  const bool hi = (lane & 4) != 0;
  // distance 4: swap the 4-column halves; afterwards the lane holds rows (j & 3) and (j & 3) + 4 of 4 columns
  const uint32_t a0 = __shfl_xor_sync(0xffffffffu, hi ? r[0] : r[2], 4);
  const uint32_t a1 = __shfl_xor_sync(0xffffffffu, hi ? r[1] : r[3], 4);
  uint32_t y0 = hi ? a0 : r[0], y1 = hi ? a1 : r[1], y2 = hi ? r[2] : a0, y3 = hi ? r[3] : a1;
  // distance 2: swap the column pairs; afterwards rows u, u+2, u+4, u+6 (u = j & 1) of one column pair
  const bool mid = (lane & 2) != 0;
  const uint32_t b0 = __shfl_xor_sync(0xffffffffu, mid ? y0 : y1, 2);
  const uint32_t b1 = __shfl_xor_sync(0xffffffffu, mid ? y2 : y3, 2);
  const uint32_t z0 = mid ? b0 : y0, z1 = mid ? y1 : b0, z2 = mid ? b1 : y2, z3 = mid ? y3 : b1;
  // distance 1: the even lane keeps the low halves (its column) and sends the high ones, the odd lane the opposite
  const bool odd = (lane & 1) != 0;
  const uint32_t c0 = __shfl_xor_sync(0xffffffffu, __byte_perm(z0, z1, odd ? 0x5410 : 0x7632), 1);
  const uint32_t c1 = __shfl_xor_sync(0xffffffffu, __byte_perm(z2, z3, odd ? 0x5410 : 0x7632), 1);
  r[0] = __byte_perm(z0, c0, odd ? 0x3254 : 0x5410);  // (row 0 | row 1) of this lane's column
  r[1] = __byte_perm(z1, c0, odd ? 0x3276 : 0x7610);  // (row 2 | row 3)
  r[2] = __byte_perm(z2, c1, odd ? 0x3254 : 0x5410);  // (row 4 | row 5)
  r[3] = __byte_perm(z3, c1, odd ? 0x3276 : 0x7610);  // (row 6 | row 7)
}

// grow0 = first key of the warp (a multiple of 32); all 32 lanes of the warp must call this together.
template <int QD0>
__device__ __forceinline__ void chain_mask_prefetch_rowk(const ChainParams& p, int h, int grow0, int lane, int col0,
                                                         uint32_t (&mk)[32]) {
  const int kcol = grow0 + 8 * (lane >> 3);  // first of the 8 keys this lane reads
#pragma unroll
  for (int q = 0; q < 2; ++q) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int qi = col0 + (QD0 + q) * 32 + 8 * i + (lane & 7);
      uint4 u = make_uint4(0, 0, 0, 0);
      if (qi < p.Lq && kcol < p.Lkv)
        u = __ldg(reinterpret_cast<const uint4*>(p.mask + (static_cast<size_t>(h) * p.Lq + qi) * p.Lkv + kcol));
      uint32_t r[4] = {u.x, u.y, u.z, u.w};
      chain_transpose8x8_b16(r, lane);
#pragma unroll
      for (int n = 0; n < 4; ++n) mk[q * 16 + 4 * i + n] = r[n];
    }
  }
}

template <bool BF16>
__device__ __forceinline__ uint64_t chain_unpack_pair(uint32_t packed) {
  if constexpr (BF16) {
    return f2_pack(__uint_as_float(packed << 16), __uint_as_float(packed & 0xffff0000u));
  } else {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&packed));
    return f2_pack(f.x, f.y);
  }
}

// W = Z * rowf * M with a mask tensor (mk: this thread's 64 mask values, packed in pairs, fetched ahead of the wait
// for Z), no shared-memory reads; the forward accumulates sum |W|. RowK: times 1/r of the column, which travels by
// shuffle from colf0 / colf1 (one column per lane and chunk) as in chain_ew_decay2.
// Config 4 with a mask tensor: forward 0.31 against 0.35 ms with the loads issued after the wait.
template <int MODE, bool BF16, int QD0, bool SPLITW>
__device__ __forceinline__ void chain_ew_mask2(uint32_t tz, const uint32_t (&mk)[32], float rowf, float colf0, float colf1,
                                               float& rsum) {
  uint32_t zr[2][32];
  tmem_ld32(tz + QD0 * 32, zr[0]);
  tmem_ld32(tz + (QD0 + 1) * 32, zr[1]);
  const uint64_t rf2 = f2_pack(rowf, rowf);
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  tc_wait_ld();
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    uint32_t pk[16];
    const float colf = q == 0 ? colf0 : colf1;
#pragma unroll
    for (int c4 = 0; c4 < 8; ++c4) {
      uint64_t a = fmul2(f2_pack(__uint_as_float(zr[q][4 * c4]), __uint_as_float(zr[q][4 * c4 + 1])), rf2);
      uint64_t b = fmul2(f2_pack(__uint_as_float(zr[q][4 * c4 + 2]), __uint_as_float(zr[q][4 * c4 + 3])), rf2);
      a = fmul2(a, chain_unpack_pair<BF16>(mk[q * 16 + 2 * c4]));
      b = fmul2(b, chain_unpack_pair<BF16>(mk[q * 16 + 2 * c4 + 1]));
      if (MODE == kChainRowK) {
        const float fa = __shfl_sync(0xffffffffu, colf, 4 * c4), fb = __shfl_sync(0xffffffffu, colf, 4 * c4 + 1);
        const float fc = __shfl_sync(0xffffffffu, colf, 4 * c4 + 2), fd = __shfl_sync(0xffffffffu, colf, 4 * c4 + 3);
        a = fmul2(a, f2_pack(fa, fb));
        b = fmul2(b, f2_pack(fc, fd));
      }
      float w0, w1, w2, w3;
      f2_unpack(a, w0, w1);
      f2_unpack(b, w2, w3);
      if (MODE == kChainFwd) {
        s0 += fabsf(w0);
        s1 += fabsf(w1);
        s2 += fabsf(w2);
        s3 += fabsf(w3);
      }
      pk[2 * c4] = pack2<BF16>(w0, w1);
      pk[2 * c4 + 1] = pack2<BF16>(w2, w3);
    }
    if constexpr (MODE == kChainFwd && !BF16) chain_check_saturation((s0 + s1) + (s2 + s3), pk);
    tmem_st16(tz + (SPLITW ? (QD0 >> 1) * 64 + q * 16 : (QD0 + q) * 16), pk);
  }
  if (MODE == kChainFwd) rsum += (s0 + s1) + (s2 + s3);
}

}  // namespace ab200
