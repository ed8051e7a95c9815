// Host launcher of the flash-attention backward. Default form: fa_bwd_prep_kernel (per-query terms into the dq
// buffer), fa_bwd_kv_sm100_kernel (dK and dV), fa_bwd_sm100_kernel<dQ>, on one stream; the older form (one
// fa_bwd_sm100_kernel per gradient: dV, dK, dQ) runs for very short query sequences and on request. The reference has
// no counterpart (python/ops/attention_interface.py:38-39); the argument order follows its backward shims for RetNet
// (csrc/kernels/retnet/bwd/profile_code.py:50-115): inputs, saved forward results, gradients out.
#pragma once

#include <math.h>

#include "chain_launch.cuh"  // persistent_grid, launch_maybe_overlapped
#include <stdlib.h>

#include "fa_bwd_kv_sm100.cuh"
#include "fa_bwd_sm100.cuh"
#include "host_common.cuh"

namespace ab200 {

struct FaBwdArgs {
  const void* q;     // [BH, Lq, D]
  const void* k;     // [BH, Lkv, D]
  const void* v;     // [BH, Lkv, D]
  const void* o;     // [BH, Lq, D]   forward output
  const void* dout;  // [BH, Lq, D]   gradient of the forward output
  const float* lse;  // [BH, Lq]      log-sum-exp written by the forward
  void* dq;          // [BH, Lq, D]
  void* dk;          // [BH, Lkv, D]
  void* dv;          // [BH, Lkv, D]
  int BH, Lq, Lkv, d;
  float scale;
  int causal;
};

template <class Cfg>
int fa_bwd_one(const void* R1, const void* R2, int r_len, const void* C1, const void* C2, const void* T, int c_len,
               FaBwdParams p, int BH, cudaStream_t stream, const char* what, bool overlap) {
  CUtensorMap tr1, tr2, tc1, tc2, tt;
  int rc;
  if ((rc = bind_device_of(R1, what))) return rc;
  if ((rc = make_tmap_3d(&tr1, R1, Cfg::BF16, Cfg::D, r_len, BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tr2, R2, Cfg::BF16, Cfg::D, r_len, BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tc1, C1, Cfg::BF16, Cfg::D, c_len, BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tc2, C2, Cfg::BF16, Cfg::D, c_len, BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tt, T, Cfg::BF16, Cfg::D, c_len, BH, 64, 128))) return rc;
  auto kernel = &fa_bwd_sm100_kernel<Cfg>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(e));
  p.nrb = (r_len + 127) / 128;
  const long long total = static_cast<long long>(p.nrb) * BH;
  if (total > 0x7fffffffLL) return fail(kErrInvalidArgument, "%s: too many tiles", what);
  p.total_items = static_cast<int>(total);
  e = launch_maybe_overlapped(kernel, persistent_grid(BH * ((p.nrb + 1) / 2)), Cfg::NTHREADS, Cfg::SMEM_BYTES, stream, overlap,
                              tr1, tr2, tc1, tc2, tt, p);
  if (e != cudaSuccess) return fail(kErrCuda, "%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
}

// dK and dV in one kernel. The per-query terms (16 bytes per query, padded to whole blocks of 128 queries) are written
// into the dq buffer by a small kernel first; dq itself is written last, by the dQ kernel.
template <int D, bool BF16>
int fa_bwd_kv_launch(const FaBwdArgs& a, cudaStream_t stream) {
  using Cfg = FaBwdKvConfig<D, BF16>;
  const char* what = "fa_bwd dK/dV";
  int rc;
  if ((rc = bind_device_of(a.k, what))) return rc;
  const int nqb = (a.Lq + 127) / 128;
  fa_bwd_prep_kernel<D, BF16><<<dim3(nqb, a.BH), 128, 0, stream>>>(a.o, a.dout, a.lse, reinterpret_cast<uint4*>(a.dq), a.Lq,
                                                                   nqb, a.scale);
  if ((rc = check_launch("fa_bwd terms"))) return rc;
  CUtensorMap tk, tv, tq, tdo;
  if ((rc = make_tmap_3d(&tk, a.k, BF16, D, a.Lkv, a.BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tv, a.v, BF16, D, a.Lkv, a.BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tq, a.q, BF16, D, a.Lq, a.BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tdo, a.dout, BF16, D, a.Lq, a.BH, 64, 128))) return rc;
  auto kernel = &fa_bwd_kv_sm100_kernel<Cfg>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "%s: cudaFuncSetAttribute: %s", what, cudaGetErrorString(e));
  FaBwdKvParams p{};
  p.dk = a.dk;
  p.dv = a.dv;
  p.terms = reinterpret_cast<const uint4*>(a.dq);
  p.Lq = a.Lq;
  p.Lkv = a.Lkv;
  p.nqb = nqb;
  p.scale = a.scale;
  p.causal = a.causal ? 1 : 0;
  p.nrb = (a.Lkv + 127) / 128;
  const long long total = static_cast<long long>(p.nrb) * a.BH;
  if (total > 0x7fffffffLL) return fail(kErrInvalidArgument, "%s: too many tiles", what);
  p.total_items = static_cast<int>(total);
  e = launch_maybe_overlapped(kernel, persistent_grid(a.BH * ((p.nrb + 1) / 2)), Cfg::NTHREADS, Cfg::SMEM_BYTES, stream, false,
                              tk, tv, tq, tdo, p);
  if (e != cudaSuccess) return fail(kErrCuda, "%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
}

// ATTN_B200_FA_BWD_SPLIT=1 in the environment selects the three-kernel backward (dV, dK, dQ) for every shape.
inline bool fa_bwd_split_requested() {
  const char* s = getenv("ATTN_B200_FA_BWD_SPLIT");
  return s != nullptr && s[0] != '\0' && s[0] != '0';
}

template <int D, bool BF16>
int fa_bwd_launch(const FaBwdArgs& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || !a.o || !a.dout || !a.lse || !a.dq || !a.dk || !a.dv)
    return fail(kErrInvalidArgument, "fa_bwd: null tensor pointer");
  if (a.BH <= 0 || a.Lq <= 0 || a.Lkv <= 0) return fail(kErrInvalidArgument, "fa_bwd: sizes must be positive");
  if (a.BH > 65535) return fail(kErrInvalidArgument, "fa_bwd: batch*heads %d exceeds 65535", a.BH);
  if (a.d != D) return fail(kErrUnsupported, "fa_bwd: head dimension %d does not match tile %d", a.d, D);
  if (a.causal && a.Lq != a.Lkv) return fail(kErrUnsupported, "fa_bwd: causal needs Lq == Lkv (got %d, %d)", a.Lq, a.Lkv);
  if (!isfinite(a.scale) || a.scale == 0.f) return fail(kErrInvalidArgument, "fa_bwd: scale must be finite and non-zero");
  const void* ptrs[] = {a.q, a.k, a.v, a.o, a.dout, a.dq, a.dk, a.dv};
  for (const void* ptr : ptrs)
    if (!aligned32(ptr)) return fail(kErrInvalidArgument, "fa_bwd: tensors must be 32-byte aligned");
  if (int prior = check_prior_status("fa_bwd")) return prior;
  FaBwdParams p{};
  p.lse = a.lse;
  p.o = a.o;
  p.dout = a.dout;
  p.Lq = a.Lq;
  p.Lkv = a.Lkv;
  p.scale = a.scale;
  p.causal = a.causal ? 1 : 0;
  FaBwdParams pv = p, pk = p, pq = p;
  pv.out = a.dv;
  pk.out = a.dk;
  pq.out = a.dq;
  // The fused dK/dV kernel parks 16 bytes per query (whole blocks of 128) in the dq buffer; that fits unless Lq is
  // tiny (less than 16 queries at d = 64, 8 at d = 128), where the three-kernel form runs instead.
  const bool fused_kv = static_cast<size_t>((a.Lq + 127) / 128) * 2048u <= static_cast<size_t>(a.Lq) * D * 2u && !fa_bwd_split_requested();
  if (fused_kv) {
    if (int rc = fa_bwd_kv_launch<D, BF16>(a, stream)) return rc;
    return fa_bwd_one<FaBwdConfig<D, kFaBwdDQ, BF16>>(a.q, a.dout, a.Lq, a.k, a.v, a.k, a.Lkv, pq, a.BH, stream, "fa_bwd dQ", true);
  }
  // unused operand slots of the dV kernel get valid maps of the used ones
  int rc = fa_bwd_one<FaBwdConfig<D, kFaBwdDV, BF16>>(a.k, a.k, a.Lkv, a.q, a.q, a.dout, a.Lq, pv, a.BH, stream, "fa_bwd dV", false);
  if (rc) return rc;
  rc = fa_bwd_one<FaBwdConfig<D, kFaBwdDK, BF16>>(a.k, a.v, a.Lkv, a.q, a.dout, a.q, a.Lq, pk, a.BH, stream, "fa_bwd dK", true);
  if (rc) return rc;
  return fa_bwd_one<FaBwdConfig<D, kFaBwdDQ, BF16>>(a.q, a.dout, a.Lq, a.k, a.v, a.k, a.Lkv, pq, a.BH, stream, "fa_bwd dQ", true);
}

}  // namespace ab200
