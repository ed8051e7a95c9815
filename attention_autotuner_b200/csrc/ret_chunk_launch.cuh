// Host launcher of the chunkwise RetNet forward (ret_chunk_sm100.cuh): argument checks, tensor maps, grid. Plays the role of the reference's retnet_recurrent_fwd
// (csrc/kernels/retnet/recurrent/recurrent.h:427-463), which fills a Params struct and launches its scan kernel.
#pragma once

#include <math.h>

#include "host_common.cuh"
#include "ret_chunk_sm100.cuh"

namespace ab200 {

struct RetChunkArgs {
  const void* q;        // [BH, L, dqk]
  const void* k;        // [BH, L, dqk]
  const void* v;        // [BH, L, dv]
  const float* decay;   // [H] per-head gamma in (0, 1]
  void* o;              // [BH, L, dv]
  int BH, H, L, dqk, dv;
  float scale;
};

inline int ret_chunk_check(const RetChunkArgs& a) {
  if (!a.q || !a.k || !a.v || !a.o || !a.decay) return fail(kErrInvalidArgument, "ret_chunk_fwd: null tensor pointer");
  if (a.BH <= 0 || a.H <= 0 || a.BH % a.H != 0 || a.L <= 0)
    return fail(kErrInvalidArgument, "ret_chunk_fwd: sizes must be positive and BH a multiple of H");
  if (a.BH > 65535) return fail(kErrInvalidArgument, "ret_chunk_fwd: batch*heads %d exceeds 65535", a.BH);
  if (a.dqk != 128 && a.dqk != 256)
    return fail(kErrUnsupported, "ret_chunk_fwd: dqk=%d (the state tile needs 128 or 256)", a.dqk);
  if (a.dv % 64 != 0 || a.dv <= 0 || a.dv > 512) return fail(kErrUnsupported, "ret_chunk_fwd: dv=%d (multiple of 64, <= 512)", a.dv);
  if (!isfinite(a.scale) || a.scale == 0.f) return fail(kErrInvalidArgument, "ret_chunk_fwd: scale must be finite and non-zero");
  if (!aligned16(a.q) || !aligned16(a.k) || !aligned16(a.v) || !aligned32(a.o))
    return fail(kErrInvalidArgument, "ret_chunk_fwd: inputs must be 16-byte aligned and the output 32-byte aligned");
  return kOk;
}

template <int DQK, int DVC, bool BF16>
int ret_chunk_launch(const RetChunkArgs& a, cudaStream_t stream) {
  using Cfg = RetChunkConfig<DQK, DVC, BF16>;
  int rc = ret_chunk_check(a);
  if (rc) return rc;
  if (a.dqk != DQK || a.dv % DVC != 0)
    return fail(kErrUnsupported, "ret_chunk_fwd: dqk=%d dv=%d do not match tile %d/%d", a.dqk, a.dv, DQK, DVC);
  if ((rc = check_prior_status("ret_chunk_fwd"))) return rc;
  if ((rc = bind_device_of(a.q, "ret_chunk_fwd"))) return rc;
  CUtensorMap tq, tk, tv;
  if ((rc = make_tmap_3d(&tq, a.q, BF16, DQK, a.L, a.BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tk, a.k, BF16, DQK, a.L, a.BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tv, a.v, BF16, a.dv, a.L, a.BH, 64, 128))) return rc;
  RetChunkParams p;
  p.o = a.o;
  p.decay = a.decay;
  p.H = a.H;
  p.L = a.L;
  p.dv = a.dv;
  p.scale = a.scale;
  auto kernel = &ret_chunk_sm100_kernel<Cfg>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "ret_chunk_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  dim3 grid(a.dv / DVC, a.BH, 1);
  kernel<<<grid, Cfg::NTHREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return check_launch("ret_chunk_fwd launch");
}

// Tile choice: 128 columns of V per CTA where dv allows it, 64 when that would leave most SMs without a CTA (a CTA walks
// its slice sequentially, so the grid BH * dv / DVC is all the parallelism there is).
template <bool BF16>
int ret_chunk_dispatch(const RetChunkArgs& a, cudaStream_t stream) {
  const bool wide = (a.dv % 128 == 0) && (static_cast<long long>(a.BH) * (a.dv / 128) >= 100);
  if (a.dqk == 128) return wide ? ret_chunk_launch<128, 128, BF16>(a, stream) : ret_chunk_launch<128, 64, BF16>(a, stream);
  if (a.dqk == 256) return wide ? ret_chunk_launch<256, 128, BF16>(a, stream) : ret_chunk_launch<256, 64, BF16>(a, stream);
  return fail(kErrUnsupported, "ret_chunk_fwd: dqk=%d (the state tile needs 128 or 256)", a.dqk);
}

}  // namespace ab200
