// Host launchers of chain_sm100_kernel for the RetNet parallel forward and backward.
// They play the role of the reference's generated launch shims
// (csrc/kernels/retnet/regfuse/profile_code.py:30-80, csrc/kernels/retnet/bwd/profile_code.py:50-115).
#pragma once

#include <math.h>

#include <type_traits>

#include "chain_pair_sm100.cuh"
#include "chain_sm100.cuh"
#include "fa_fwd_launch.cuh"  // profile_loop
#include "host_common.cuh"

namespace ab200 {

struct RetArgs {
  const void* q;     // [BH, Lq, dqk]
  const void* k;     // [BH, Lkv, dqk]
  const void* v;     // [BH, Lkv, dv]
  const void* mask;  // [H, Lq, Lkv] 16-bit, or nullptr when decay is given
  const float* decay;  // [H] gammas (device), or nullptr when mask is given
  // forward
  void* o;           // [BH, Lq, dv]
  float* r;          // [BH, Lq]   written by forward, read by backward
  // backward
  const void* dout;  // [BH, Lq, dv]
  void* dq;          // [BH, Lq, dqk]
  void* dk;          // [BH, Lkv, dqk]
  void* dv_out;      // [BH, Lkv, dv]
  // backward with a mask tensor: optional scratch for a transposed copy of the mask (H * Lq * Lkv 16-bit values,
  // 16-byte aligned); nullptr or too small: the kernels read columns of the mask and transpose them in registers
  void* workspace;
  size_t workspace_bytes;
  int BH, H, Lq, Lkv, dqk, dv;
  float scale;
  int causal;        // with a general mask: 1 = mask is lower triangular, skip the blocks above the diagonal
};

inline int ret_check_common(const RetArgs& a, const char* what) {
  if (!a.q || !a.k || !a.v) return fail(kErrInvalidArgument, "%s: null tensor pointer", what);
  if ((a.mask == nullptr) == (a.decay == nullptr))
    return fail(kErrInvalidArgument, "%s: exactly one of mask / decay must be given", what);
  if (a.BH <= 0 || a.H <= 0 || a.BH % a.H != 0 || a.Lq <= 0 || a.Lkv <= 0)
    return fail(kErrInvalidArgument, "%s: sizes must be positive and BH a multiple of H", what);
  if (a.BH > 65535) return fail(kErrInvalidArgument, "%s: batch*heads %d exceeds 65535", what, a.BH);
  if (a.mask && a.Lkv % 8 != 0) return fail(kErrUnsupported, "%s: a mask tensor needs Lkv %% 8 == 0 (got %d)", what, a.Lkv);
  if (!isfinite(a.scale) || a.scale == 0.f) return fail(kErrInvalidArgument, "%s: scale must be finite and non-zero", what);
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || (a.mask && !aligned16(a.mask)))
    return fail(kErrInvalidArgument, "%s: tensors must be 16-byte aligned", what);
  return check_prior_status(what);
}

// CTAs of the persistent grid: one per SM (a CTA uses all of shared and tensor memory). The kernels hand out
// equal-cost pairs of row blocks round-robin, so any grid size is balanced.
inline int persistent_grid(int n_super) {
  static int sms = [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      n = 148;
    return n > 0 ? n : 148;
  }();
  return n_super < sms ? n_super : sms;
}

// Launch helper: `overlap` marks the kernel as a programmatic dependent of the previous kernel in the stream (it may
// start while that one drains; the kernels wait for it before they complete).
#ifndef AB200_PDL
#define AB200_PDL 1
#endif
template <class Kernel, class... Args>
cudaError_t launch_maybe_overlapped(Kernel kernel, int grid, int block, int smem, cudaStream_t stream, bool overlap, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(block, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = (overlap && AB200_PDL) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

// One launch of the chain kernel. r_len / c_len are the lengths of the row / column side; k1 and n2_total
// the inner extents of the R/C and T tensors.
template <class Cfg>
int chain_launch(const void* R, int r_len, const void* C, int c_len, const void* T, int n2_total, ChainParams p, int BH,
                 cudaStream_t stream, const char* what, bool overlap = false) {
  CUtensorMap tr, tc, tt;
  int rc;
  if (!aligned32(p.out)) return fail(kErrInvalidArgument, "%s: output tensors must be 32-byte aligned", what);
  if ((rc = bind_device_of(R, what))) return rc;
  if ((rc = make_tmap_3d(&tr, R, Cfg::BF16, Cfg::K1, r_len, BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tc, C, Cfg::BF16, Cfg::K1, c_len, BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tt, T, Cfg::BF16, n2_total, c_len, BH, 64, 128))) return rc;
  auto kernel = &chain_sm100_kernel<Cfg>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(e));
  p.nrb = (r_len + 127) / 128;
  p.ny = n2_total / Cfg::N2;
  const long long total = static_cast<long long>(p.nrb) * p.ny * BH;
  if (total > 0x7fffffffLL) return fail(kErrInvalidArgument, "%s: too many tiles", what);
  p.total_items = static_cast<int>(total);
  e = launch_maybe_overlapped(kernel, persistent_grid((p.total_items / p.nrb) * ((p.nrb + 1) / 2)), Cfg::NTHREADS,
                              Cfg::SMEM_BYTES, stream, overlap, tr, tc, tt, p);
  if (e != cudaSuccess) return fail(kErrCuda, "%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
}

// One launch of the CTA-pair chain kernel: clusters of two CTAs, each cluster a 256-row tile. The persistent grid
// holds as many clusters as can be resident at once (asked from the occupancy API, since pairs need both SMs
// of a TPC).
template <class Cfg>
int chain_pair_launch(const void* R, int r_len, const void* C, int c_len, const void* T, int n2_total, ChainParams p, int BH,
                      cudaStream_t stream, const char* what, bool overlap = false) {
  CUtensorMap tr, tc, tt, to;
  int rc;
  if (!aligned32(p.out)) return fail(kErrInvalidArgument, "%s: output tensors must be 32-byte aligned", what);
  if ((rc = bind_device_of(R, what))) return rc;
  if ((rc = make_tmap_3d(&tr, R, Cfg::BF16, Cfg::K1, r_len, BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tc, C, Cfg::BF16, Cfg::K1, c_len, BH, 64, 64))) return rc;
  if ((rc = make_tmap_3d(&tt, T, Cfg::BF16, n2_total, c_len, BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&to, p.out, Cfg::BF16, p.ld_out, r_len, BH, 64, 128))) return rc;
  auto kernel = &chain_pair_sm100_kernel<Cfg>;
  // The attribute belongs to this library's copy of the kernel and is set on every launch: a function-local
  // static of a template is one object per PROCESS (unique symbol), shared by every loaded library that holds
  // the same instantiation, so it may only cache what is the same for all of them (the occupancy answer).
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(e));
  static int max_clusters = 0;
  if (max_clusters == 0) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(2, 1, 1);
    cfg.blockDim = dim3(Cfg::NTHREADS, 1, 1);
    cfg.dynamicSmemBytes = Cfg::SMEM_BYTES;
    cudaLaunchAttribute attr{};
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kernel, &cfg);
    if (e != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      return fail(kErrCuda, "%s: no CTA pair can be resident (%s)", what, e != cudaSuccess ? cudaGetErrorString(e) : "0 clusters");
    }
    max_clusters = n;
  }
  p.nrb = (r_len + 255) / 256;
  p.ny = n2_total / Cfg::N2;
  const long long total = static_cast<long long>(p.nrb) * p.ny * BH;
  if (total > 0x7fffffffLL) return fail(kErrInvalidArgument, "%s: too many tiles", what);
  p.total_items = static_cast<int>(total);
  // equal-cost super-items (pairs of row blocks) are handed out round-robin: any number of clusters is balanced
  const int n_super = (p.total_items / p.nrb) * ((p.nrb + 1) / 2);
  const int clusters = n_super < max_clusters ? n_super : max_clusters;
  e = launch_maybe_overlapped(kernel, 2 * clusters, Cfg::NTHREADS, Cfg::SMEM_BYTES, stream, overlap, tr, tc, tt, to, p);
  if (e != cudaSuccess) return fail(kErrCuda, "%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
}

inline ChainParams ret_params(const RetArgs& a) {
  ChainParams p{};
  p.mask = reinterpret_cast<const uint16_t*>(a.mask);
  p.decay = a.decay;
  p.H = a.H;
  p.Lq = a.Lq;
  p.Lkv = a.Lkv;
  p.scale = a.scale;
  p.skip_upper = (a.decay != nullptr || a.causal) ? 1 : 0;
  return p;
}

// Launch of either family: PAIR = true runs the CTA-pair kernel (N2 must be 128 or 256).
template <bool PAIR, int K1, int N2, int MODE, bool GENERAL, bool BF16>
int chain_go(const void* R, int r_len, const void* C, int c_len, const void* T, int n2_total, const ChainParams& p, int BH,
             cudaStream_t stream, const char* what, bool overlap = false) {
  if constexpr (PAIR) {
    return chain_pair_launch<ChainPairConfig<K1, N2, MODE, GENERAL, BF16>>(R, r_len, C, c_len, T, n2_total, p, BH, stream, what,
                                                                           overlap);
  } else {
    return chain_launch<ChainConfig<K1, N2, MODE, GENERAL, BF16>>(R, r_len, C, c_len, T, n2_total, p, BH, stream, what, overlap);
  }
}

// Forward. DQK = head dim of q/k, DVC = columns of V per CTA or CTA pair (divides dv).
template <int DQK, int DVC, bool BF16, bool PAIR = false>
int ret_fwd_launch(const RetArgs& a, cudaStream_t stream) {
  int rc = ret_check_common(a, "ret_fwd");
  if (rc) return rc;
  if (!a.o || !a.r) return fail(kErrInvalidArgument, "ret_fwd: null output pointer");
  if (a.dqk != DQK || a.dv % DVC != 0) return fail(kErrUnsupported, "ret_fwd: dqk=%d dv=%d do not match tile %d/%d", a.dqk, a.dv, DQK, DVC);
  ChainParams p = ret_params(a);
  p.out = a.o;
  p.ld_out = a.dv;
  p.r_out = a.r;
  if (a.mask)
    return chain_go<PAIR, DQK, DVC, kChainFwd, true, BF16>(a.q, a.Lq, a.k, a.Lkv, a.v, a.dv, p, a.BH, stream, "ret_fwd");
  return chain_go<PAIR, DQK, DVC, kChainFwd, false, BF16>(a.q, a.Lq, a.k, a.Lkv, a.v, a.dv, p, a.BH, stream, "ret_fwd");
}

// Backward: dV, dK, dQ as three launches on the same stream. DV = full head dim of v (contraction length
// of the dK and dQ kernels), DVC / DQC = output columns per CTA of the dV kernel / of the dK and dQ kernels.
template <int DQK, int DV, int DVC, int DQC, bool BF16, bool PAIR = false>
int ret_bwd_launch(const RetArgs& a, cudaStream_t stream) {
  int rc = ret_check_common(a, "ret_bwd");
  if (rc) return rc;
  if (!a.dout || !a.r || !a.dq || !a.dk || !a.dv_out) return fail(kErrInvalidArgument, "ret_bwd: null pointer");
  if (a.dqk != DQK || a.dv != DV) return fail(kErrUnsupported, "ret_bwd: dqk=%d dv=%d do not match tile %d/%d", a.dqk, a.dv, DQK, DV);
  static_assert(DV % DVC == 0 && DQK % DQC == 0, "chunking");
  ChainParams p = ret_params(a);
  p.r_in = a.r;
  // Mask tensor: the dV and dK kernels own keys and need columns of M[h][query][key]. With scratch memory at hand the
  // mask is transposed once per call (one coalesced pass over H * Lq * Lkv values) and those kernels read rows of the
  // copy with 16-byte loads; without it every warp reads 32 x 32 tiles by rows and transposes them in registers
  // (three shuffle rounds per 8 x 8 block, on the element-wise warps' critical path).
  const size_t mask_bytes = static_cast<size_t>(a.H) * a.Lq * a.Lkv * 2u;
  const uint16_t* mask_t = nullptr;
  if (a.mask && a.workspace && aligned16(a.workspace) && a.workspace_bytes >= mask_bytes && a.Lq % 8 == 0) {
    dim3 tgrid((a.Lkv + 31) / 32, (a.Lq + 31) / 32, a.H);
    mask_transpose_kernel<<<tgrid, dim3(32, 8, 1), 0, stream>>>(reinterpret_cast<const uint16_t*>(a.mask),
                                                              reinterpret_cast<uint16_t*>(a.workspace), a.Lq, a.Lkv);
    if ((rc = check_launch("ret_bwd mask transpose"))) return rc;
    mask_t = reinterpret_cast<const uint16_t*>(a.workspace);
  }
  auto go = [&](auto general_tag) -> int {
    constexpr bool G = decltype(general_tag)::value;
    ChainParams pv = p;
    pv.out = a.dv_out;
    pv.ld_out = a.dv;
    pv.mask_t = mask_t;
    int r1 = chain_go<PAIR, DQK, DVC, kChainRowK, G, BF16>(a.k, a.Lkv, a.q, a.Lq, a.dout, a.dv, pv, a.BH, stream, "ret_bwd dV");
    if (r1) return r1;
    ChainParams pk = p;
    pk.out = a.dk;
    pk.ld_out = a.dqk;
    pk.mask_t = mask_t;
    r1 = chain_go<PAIR, DV, DQC, kChainRowK, G, BF16>(a.v, a.Lkv, a.dout, a.Lq, a.q, a.dqk, pk, a.BH, stream, "ret_bwd dK", true);
    if (r1) return r1;
    ChainParams pq = p;
    pq.out = a.dq;
    pq.ld_out = a.dqk;
    return chain_go<PAIR, DV, DQC, kChainRowQ, G, BF16>(a.dout, a.Lq, a.v, a.Lkv, a.k, a.dqk, pq, a.BH, stream, "ret_bwd dQ", true);
  };
  return a.mask ? go(std::true_type{}) : go(std::false_type{});
}

}  // namespace ab200
