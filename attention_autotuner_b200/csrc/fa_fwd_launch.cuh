// Host launcher for fa_fwd_sm100_kernel: argument checks, tensor maps, grid, timing loop.
// Plays the role of the reference's generated launch shims
// (csrc/kernels/attention/regfuse/profile_code.py:28-76: profile() and kernel_entry()).
#pragma once

#include <math.h>

#include <stdlib.h>

#include "fa_fwd_pair_sm100.cuh"
#include "fa_fwd_persist_sm100.cuh"
#include "fa_fwd_sm100.cuh"
#include "host_common.cuh"

namespace ab200 {

struct FaFwdArgs {
  const void* q;  // [BH, Lq, dqk]
  const void* k;  // [BH, Lkv, dqk]
  const void* v;  // [BH, Lkv, dv]
  void* o;        // [BH, Lq, dv]
  float* lse;     // [BH, Lq] or nullptr
  int BH, Lq, Lkv, dv;
  float scale;
  int causal;
};

template <class Cfg>
int fa_fwd_launch(const FaFwdArgs& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || !a.o) return fail(kErrInvalidArgument, "fa_fwd: null tensor pointer");
  if (a.BH <= 0 || a.Lq <= 0 || a.Lkv <= 0) return fail(kErrInvalidArgument, "fa_fwd: sizes must be positive");
  if (a.BH > 65535) return fail(kErrInvalidArgument, "fa_fwd: batch*heads %d exceeds 65535", a.BH);
  if (a.dv % Cfg::DV != 0) return fail(kErrUnsupported, "fa_fwd: dv %d is not a multiple of the tile's %d", a.dv, Cfg::DV);
  if (!(a.scale > 0.f) || !isfinite(a.scale)) return fail(kErrInvalidArgument, "fa_fwd: scale must be positive and finite");
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned32(a.o))
    return fail(kErrInvalidArgument, "fa_fwd: inputs must be 16-byte aligned and the output 32-byte aligned");

  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = check_prior_status("fa_fwd"))) return rc;
  if ((rc = bind_device_of(a.q, "fa_fwd"))) return rc;
  if ((rc = make_tmap_3d(&tq, a.q, Cfg::BF16, Cfg::DQK, a.Lq, a.BH, 64, Cfg::BM))) return rc;
  if ((rc = make_tmap_3d(&tk, a.k, Cfg::BF16, Cfg::DQK, a.Lkv, a.BH, 64, Cfg::BN))) return rc;
  if ((rc = make_tmap_3d(&tv, a.v, Cfg::BF16, a.dv, a.Lkv, a.BH, 64, Cfg::BN))) return rc;

  FaFwdParams p;
  p.o = a.o;
  p.lse = a.lse;
  p.dv_total = a.dv;
  p.Lq = a.Lq;
  p.Lkv = a.Lkv;
  p.causal = a.causal ? 1 : 0;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;

  auto kernel = &fa_fwd_sm100_kernel<Cfg>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "fa_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  dim3 grid((a.Lq + Cfg::BM * Cfg::NQ - 1) / (Cfg::BM * Cfg::NQ), a.dv / Cfg::DV, a.BH);
  kernel<<<grid, Cfg::NTHREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return check_launch("fa_fwd launch");
}

// ATTN_B200_FA_FWD_FORM in the environment overrides the choice between the two forms of the kernel for every shape
// they both cover: "grid" (one CTA per 256 query rows) or "persistent" (one CTA per SM walking a work list).
inline int fa_fwd_form_requested() {  // 0: automatic, 1: grid, 2: persistent
  const char* s = getenv("ATTN_B200_FA_FWD_FORM");
  if (s == nullptr) return 0;
  if (s[0] == 'g') return 1;
  if (s[0] == 'p') return 2;
  return 0;
}

// Launcher of the persistent kernel: one CTA per SM (fewer when there is less work) walking the work list.
template <class Cfg>
int fa_fwd_persist_launch(const FaFwdArgs& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || !a.o) return fail(kErrInvalidArgument, "fa_fwd: null tensor pointer");
  if (a.BH <= 0 || a.Lq <= 0 || a.Lkv <= 0) return fail(kErrInvalidArgument, "fa_fwd: sizes must be positive");
  if (a.BH > 65535) return fail(kErrInvalidArgument, "fa_fwd: batch*heads %d exceeds 65535", a.BH);
  if (a.dv % Cfg::DV != 0) return fail(kErrUnsupported, "fa_fwd: dv %d is not a multiple of the tile's %d", a.dv, Cfg::DV);
  if (!(a.scale > 0.f) || !isfinite(a.scale)) return fail(kErrInvalidArgument, "fa_fwd: scale must be positive and finite");
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned32(a.o))
    return fail(kErrInvalidArgument, "fa_fwd: inputs must be 16-byte aligned and the output 32-byte aligned");

  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = check_prior_status("fa_fwd"))) return rc;
  if ((rc = bind_device_of(a.q, "fa_fwd"))) return rc;
  if ((rc = make_tmap_3d(&tq, a.q, Cfg::BF16, Cfg::DQK, a.Lq, a.BH, 64, Cfg::BM))) return rc;
  if ((rc = make_tmap_3d(&tk, a.k, Cfg::BF16, Cfg::DQK, a.Lkv, a.BH, 64, Cfg::BN))) return rc;
  if ((rc = make_tmap_3d(&tv, a.v, Cfg::BF16, a.dv, a.Lkv, a.BH, 64, Cfg::BN))) return rc;
  CUtensorMap to = tv;  // stands in where the output is not staged
  using Lay = FaFwdPersistLayout<Cfg>;
  if (Lay::STAGE_O && (rc = make_tmap_3d(&to, a.o, Cfg::BF16, a.dv, a.Lq, a.BH, 64, 32))) return rc;  // a warp stores its 32 rows

  FaFwdPersistParams pp;
  pp.f.o = a.o;
  pp.f.lse = a.lse;
  pp.f.dv_total = a.dv;
  pp.f.Lq = a.Lq;
  pp.f.Lkv = a.Lkv;
  pp.f.causal = a.causal ? 1 : 0;
  pp.f.scale = a.scale;
  pp.f.scale_log2 = a.scale * 1.4426950408889634f;
  pp.nqb = (a.Lq + Cfg::BM * Cfg::NQ - 1) / (Cfg::BM * Cfg::NQ);
  pp.ndv = a.dv / Cfg::DV;
  const long long n_super = static_cast<long long>(a.BH) * pp.ndv * ((pp.nqb + 1) / 2);
  if (n_super > 0x3fffffffLL) return fail(kErrInvalidArgument, "fa_fwd: too many tiles");
  pp.n_super = static_cast<int>(n_super);

  auto kernel = &fa_fwd_persist_sm100_kernel<Cfg>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "fa_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const int grid = pp.n_super < sms ? pp.n_super : sms;
  kernel<<<grid, Cfg::NTHREADS, Lay::SMEM_BYTES, stream>>>(tq, tk, tv, to, pp);
  return check_launch("fa_fwd launch");
}

// The default tile (two query tiles, up to 128 V columns, no softmax variant) exists in both forms; the persistent one
// runs where a CTA's work items are short, because what it saves lies at their boundaries. Measured against the grid
// form in one session (d = 128, back-to-back launches), without a mask / under a causal one: 148 slices of L = 2048
// +5 % / +18 %, B=8 H=16 L=4096 +1 % / +8 %, L = 8192 0 % / +3 %, B=16 H=32 L=16384 -2 % / -2 %, Lq=1024 x Lkv=16384
// -3 % (with long items a static work list loses more to the slowest SM than the boundaries cost). The rule: persistent
// up to 40 KV blocks per item on average (half of the blocks count under a causal mask).
template <class Cfg>
bool fa_fwd_picks_persistent(const FaFwdArgs& a) {
  if constexpr (Cfg::NQ == 2 && Cfg::SPLIT == 1 && Cfg::NMMA == 1 && Cfg::EXP_EMU == 0 && Cfg::EXP_H2 == 0 && Cfg::DV <= 128) {
    const int form = fa_fwd_form_requested();
    const int nblk = (a.Lkv + Cfg::BN - 1) / Cfg::BN;
    const int avg_blocks = a.causal ? (nblk + 1) / 2 : nblk;
    return form == 2 || (form == 0 && avg_blocks <= 40);
  }
  return false;
}

template <class Cfg>
int fa_fwd_launch_auto(const FaFwdArgs& a, cudaStream_t stream) {
  if constexpr (Cfg::NQ == 2 && Cfg::SPLIT == 1 && Cfg::NMMA == 1 && Cfg::EXP_EMU == 0 && Cfg::EXP_H2 == 0 && Cfg::DV <= 128) {
    if (fa_fwd_picks_persistent<Cfg>(a)) return fa_fwd_persist_launch<Cfg>(a, stream);
  }
  return fa_fwd_launch<Cfg>(a, stream);
}

// Launcher of the CTA-pair kernel: clusters of two CTAs along x, each cluster a 512-row block of queries.
template <class Cfg>
int fa_fwd_pair_launch(const FaFwdArgs& a, cudaStream_t stream) {
  if (!a.q || !a.k || !a.v || !a.o) return fail(kErrInvalidArgument, "fa_fwd: null tensor pointer");
  if (a.BH <= 0 || a.Lq <= 0 || a.Lkv <= 0) return fail(kErrInvalidArgument, "fa_fwd: sizes must be positive");
  if (a.BH > 65535) return fail(kErrInvalidArgument, "fa_fwd: batch*heads %d exceeds 65535", a.BH);
  if (a.dv % Cfg::DV != 0) return fail(kErrUnsupported, "fa_fwd: dv %d is not a multiple of the tile's %d", a.dv, Cfg::DV);
  if (!(a.scale > 0.f) || !isfinite(a.scale)) return fail(kErrInvalidArgument, "fa_fwd: scale must be positive and finite");
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned32(a.o))
    return fail(kErrInvalidArgument, "fa_fwd: inputs must be 16-byte aligned and the output 32-byte aligned");

  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = check_prior_status("fa_fwd"))) return rc;
  if ((rc = bind_device_of(a.q, "fa_fwd"))) return rc;
  if ((rc = make_tmap_3d(&tq, a.q, Cfg::BF16, Cfg::DQK, a.Lq, a.BH, 64, Cfg::BM))) return rc;
  if ((rc = make_tmap_3d(&tk, a.k, Cfg::BF16, Cfg::DQK, a.Lkv, a.BH, 64, Cfg::BN / 2))) return rc;  // half of the keys
  if ((rc = make_tmap_3d(&tv, a.v, Cfg::BF16, a.dv, a.Lkv, a.BH, 64, Cfg::BN))) return rc;          // half of the columns

  FaFwdParams p;
  p.o = a.o;
  p.lse = a.lse;
  p.dv_total = a.dv;
  p.Lq = a.Lq;
  p.Lkv = a.Lkv;
  p.causal = a.causal ? 1 : 0;
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;

  auto kernel = &fa_fwd_pair_sm100_kernel<Cfg>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "fa_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const int rows_per_pair = 2 * Cfg::BM * Cfg::NQ;
  dim3 grid(2 * ((a.Lq + rows_per_pair - 1) / rows_per_pair), a.dv / Cfg::DV, a.BH);
  kernel<<<grid, Cfg::NTHREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return check_launch("fa_fwd launch");
}

// One warm-up launch, then enough launches to fill about 100 ms; returns ms per launch, -1 on error.
template <class F>
float profile_loop(F&& launch_once, cudaStream_t stream) {
  cudaEvent_t e0, e1;
  if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return -1.f;
  float ms = -1.f;
  do {
    cudaEventRecord(e0, stream);
    if (launch_once() != kOk) break;
    if (cudaEventRecord(e1, stream) != cudaSuccess || cudaEventSynchronize(e1) != cudaSuccess) break;
    float t = 0.f;
    cudaEventElapsedTime(&t, e0, e1);
    int repeats = t > 0.f ? static_cast<int>(ceilf(100.0f / t)) : 100;
    if (repeats < 1) repeats = 1;
    if (repeats > 2000) repeats = 2000;
    cudaEventRecord(e0, stream);
    bool bad = false;
    for (int i = 0; i < repeats; ++i)
      if (launch_once() != kOk) { bad = true; break; }
    if (bad) break;
    if (cudaEventRecord(e1, stream) != cudaSuccess || cudaEventSynchronize(e1) != cudaSuccess) break;
    if (cudaGetLastError() != cudaSuccess) break;
    cudaEventElapsedTime(&t, e0, e1);
    int det = 0;
    if (read_device_status(1, &det) != 0) break;
    ms = t / repeats;
  } while (0);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  return ms;
}

}  // namespace ab200
