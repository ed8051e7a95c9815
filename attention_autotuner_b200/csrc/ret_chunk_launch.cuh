// Host launcher of the chunkwise RetNet forward (ret_chunk_sm100.cuh): argument checks, tensor maps, grid. Plays the role of the reference's retnet_recurrent_fwd
// (csrc/kernels/retnet/recurrent/recurrent.h:427-463), which fills a Params struct and launches its scan kernel.
#pragma once

#include <math.h>

#include <algorithm>

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
  // optional scratch for the segment states (ret_chunk_workspace_bytes); with none the sequence is walked in one piece
  void* workspace = nullptr;
  size_t workspace_bytes = 0;
  int segments = 0;     // 0: the library chooses; n > 0: exactly min(n, chunks) segments (an error if the scratch is too small)
};

// Segments the library would cut the sequence into, given room for them: as many as fill the SMs with CTAs of 128
// columns, each at least four chunks long; 1 (a walk in order) when the slices alone fill the GPU.
inline int ret_chunk_preferred_segments(int BH, int L, int dv) {
  if (dv % 128 != 0) return 1;
  const long long tiles = static_cast<long long>(BH) * (dv / 128);
  const int nchunk = (L + 127) / 128;
  const long long g = std::min<long long>(148 / std::max<long long>(tiles, 1), nchunk / 4);
  return g >= 2 ? static_cast<int>(g) : 1;
}

// Number of segments that `segments` chunks-per-piece arithmetic really yields (the last may be short), and the scratch
// they need: one fp32 state tile [dqk x dv] per slice and segment but the last.
inline int ret_chunk_segment_chunks(int L, int segments) {
  const int nchunk = (L + 127) / 128;
  const int g = std::max(1, std::min(segments, nchunk));
  return (nchunk + g - 1) / g;
}
inline int ret_chunk_segment_count(int L, int segments) {
  const int nchunk = (L + 127) / 128;
  const int seg = ret_chunk_segment_chunks(L, segments);
  return (nchunk + seg - 1) / seg;
}
inline size_t ret_chunk_workspace_bytes(int BH, int L, int dqk, int dv, int segments) {
  const int g = ret_chunk_segment_count(L, segments);
  return static_cast<size_t>(g - 1) * BH * dqk * dv * sizeof(float);
}

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
int ret_chunk_launch(const RetChunkArgs& a, cudaStream_t stream, int segments = 1) {
  using Cfg = RetChunkConfig<DQK, DVC, BF16>;
  int rc = ret_chunk_check(a);
  if (rc) return rc;
  if (a.dqk != DQK || a.dv % DVC != 0)
    return fail(kErrUnsupported, "ret_chunk_fwd: dqk=%d dv=%d do not match tile %d/%d", a.dqk, a.dv, DQK, DVC);
  if ((rc = check_prior_status("ret_chunk_fwd"))) return rc;
  if ((rc = bind_device_of(a.q, "ret_chunk_fwd"))) return rc;
  CUtensorMap tq, tk, tv, to;
  if ((rc = make_tmap_3d(&tq, a.q, BF16, DQK, a.L, a.BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tk, a.k, BF16, DQK, a.L, a.BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&tv, a.v, BF16, a.dv, a.L, a.BH, 64, 128))) return rc;
  if ((rc = make_tmap_3d(&to, a.o, BF16, a.dv, a.L, a.BH, 64, 32))) return rc;  // a warp stores its 32 rows
  RetChunkParams p;
  p.o = a.o;
  p.decay = a.decay;
  p.H = a.H;
  p.L = a.L;
  p.dv = a.dv;
  p.scale = a.scale;
  const int nseg = ret_chunk_segment_count(a.L, segments);
  p.seg = ret_chunk_segment_chunks(a.L, segments);
  p.ws = nseg > 1 ? static_cast<float*>(a.workspace) : nullptr;
  if (nseg > 65535) return fail(kErrInvalidArgument, "ret_chunk_fwd: %d segments exceed 65535", nseg);
  if (nseg > 1) {
    // the state each segment but the last leaves behind, then every segment at once
    using Lay = RetChunkStateLayout<Cfg>;
    auto state_kernel = &ret_chunk_state_sm100_kernel<Cfg>;
    cudaError_t es = cudaFuncSetAttribute(state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Lay::SMEM_BYTES);
    if (es != cudaSuccess) return fail(kErrCuda, "ret_chunk_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(es));
    dim3 sgrid(a.dv / DVC, a.BH, nseg - 1);
    state_kernel<<<sgrid, Lay::NTHREADS, Lay::SMEM_BYTES, stream>>>(tk, tv, p);
    if ((rc = check_launch("ret_chunk_fwd state launch"))) return rc;
  }
  auto kernel = &ret_chunk_sm100_kernel<Cfg>;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
  if (e != cudaSuccess) return fail(kErrCuda, "ret_chunk_fwd: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  dim3 grid(a.dv / DVC, a.BH, nseg);
  kernel<<<grid, Cfg::NTHREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, to, p);
  return check_launch("ret_chunk_fwd launch");
}

// Tile choice: 128 columns of V per CTA where dv allows it, 64 when that would leave most SMs without a CTA (a CTA walks
// its slice sequentially, so the grid BH * dv / DVC is all the parallelism there is).
template <bool BF16>
int ret_chunk_dispatch(const RetChunkArgs& a, cudaStream_t stream) {
  if (int rc = ret_chunk_check(a)) return rc;
  // Segments: asked for by number, or as many as the library prefers and the scratch holds (fewer when it is small).
  int segments = 1;
  if (a.segments < 0) return fail(kErrInvalidArgument, "ret_chunk_fwd: segments=%d", a.segments);
  if (a.segments > 0) {
    segments = ret_chunk_segment_count(a.L, a.segments);
    if (segments > 1 && (!a.workspace || !aligned16(a.workspace) ||
                         a.workspace_bytes < ret_chunk_workspace_bytes(a.BH, a.L, a.dqk, a.dv, segments)))
      return fail(kErrInvalidArgument, "ret_chunk_fwd: %d segments need %zu bytes of 16-byte aligned scratch, got %zu", segments,
                  ret_chunk_workspace_bytes(a.BH, a.L, a.dqk, a.dv, segments), a.workspace ? a.workspace_bytes : size_t(0));
  } else if (a.workspace && aligned16(a.workspace)) {
    segments = ret_chunk_preferred_segments(a.BH, a.L, a.dv);
    while (segments > 1 && a.workspace_bytes < ret_chunk_workspace_bytes(a.BH, a.L, a.dqk, a.dv, segments)) --segments;
    segments = ret_chunk_segment_count(a.L, segments);
  }
  if (segments > 1) {
    // every CTA of a segmented walk owns the widest tile dv allows: the segments, not the tile, spread the work
    const bool w = a.dv % 128 == 0;
    if (a.dqk == 128) return w ? ret_chunk_launch<128, 128, BF16>(a, stream, segments) : ret_chunk_launch<128, 64, BF16>(a, stream, segments);
    return w ? ret_chunk_launch<256, 128, BF16>(a, stream, segments) : ret_chunk_launch<256, 64, BF16>(a, stream, segments);
  }
  const bool wide = (a.dv % 128 == 0) && (static_cast<long long>(a.BH) * (a.dv / 128) >= 100);
  if (a.dqk == 128) return wide ? ret_chunk_launch<128, 128, BF16>(a, stream) : ret_chunk_launch<128, 64, BF16>(a, stream);
  if (a.dqk == 256) return wide ? ret_chunk_launch<256, 128, BF16>(a, stream) : ret_chunk_launch<256, 64, BF16>(a, stream);
  return fail(kErrUnsupported, "ret_chunk_fwd: dqk=%d (the state tile needs 128 or 256)", a.dqk);
}

}  // namespace ab200
