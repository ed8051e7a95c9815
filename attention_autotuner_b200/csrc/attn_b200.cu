// libattn_b200.so: the ahead-of-time built C-ABI library (declarations in include/attn_b200.h).
// Holds the default tile configuration of every kernel for the supported head dimensions; the
// autotuner compiles further configurations into separate per-config libraries from the same
// kernel headers.
#include "../../include/attn_b200.h"

#include <mutex>

#include "chain_launch.cuh"
#include "fa_bwd_launch.cuh"
#include "fa_fwd_launch.cuh"
#include "ret_chunk_launch.cuh"
#include "selftest.cuh"
#include "selftest_pair.cuh"

using namespace ab200;

// ---------------------------------------------------------------------------------------------------------------------
// Scratch of attn_b200_ret_bwd_noalloc: device memory that belongs to the library itself, for callers that cannot
// hand over a workspace and must not cause an allocation. A file-scope array: every device that loads this library
// holds these bytes from the moment the module is loaded until the process exits. In host code the NAME of the array is
// only a stand-in for the symbol; the address a kernel can use comes from cudaGetSymbolAddress (noalloc_scratch below).
// ---------------------------------------------------------------------------------------------------------------------
constexpr size_t kNoAllocScratchBytes = 32u << 20;  // 32 MiB: a transposed 16-bit mask of up to 16 Mi elements (H * Lq * Lkv)
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

namespace {

// Device address of g_noalloc_scratch on the calling thread's current device. Looked up once per device, with that
// device current (the first call of attn_b200_ret_bwd_noalloc on a device does it, which also binds the device's
// context to the thread), and remembered.
int noalloc_scratch(void** out) {
  constexpr int kMaxDevices = 64;
  static void* table[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(kErrCuda, "ret_bwd_noalloc: no usable current device");
  std::lock_guard<std::mutex> lock(mu);
  if (table[dev] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return fail(kErrCuda, "ret_bwd_noalloc: cudaGetSymbolAddress(scratch) on device %d: %s", dev, cudaGetErrorString(e));
    }
    table[dev] = ptr;
  }
  *out = table[dev];
  return kOk;
}

// Default flash-attention tiles per (dqk, dv-chunk): two ping-ponging query tiles when tensor memory
// and shared memory allow it, otherwise one.
template <bool BF16>
int fa_fwd_dispatch(const FaFwdArgs& a, int dqk, cudaStream_t st, bool profile, float* ms) {
  auto run = [&](auto cfg_tag) -> int {
    using Cfg = decltype(cfg_tag);
    auto launch = [&]() -> int {
      // the persistent form with a K / V ring of three entries leaves room to stage the finished tiles in shared memory
      // and store them by TMA (the tuner's choice at d = 128 as well); the grid form keeps its ring of four
      if constexpr (Cfg::DQK == 128 && Cfg::NQ == 2 && Cfg::NSTAGE == 4) {
        using P = FaFwdConfig<128, Cfg::DV, 2, 3, Cfg::BF16>;
        if (fa_fwd_picks_persistent<P>(a)) return fa_fwd_persist_launch<P>(a, st);
      }
      return fa_fwd_launch_auto<Cfg>(a, st);
    };
    if (!profile) return launch();
    *ms = profile_loop(launch, st);
    return *ms < 0.f ? kErrCuda : kOk;
  };
  // chunk of the V head dim handled per CTA
  const int dv = a.dv;
  const int chunk = (dv % 256 == 0) ? 256 : (dv % 128 == 0) ? 128 : 64;
  if (dv % 64 != 0 || dv > 512 || dv <= 0) return fail(kErrUnsupported, "fa_fwd: dv=%d (need multiple of 64, <= 512)", dv);
  switch (dqk) {
    case 64:
      if (chunk == 64) return run(FaFwdConfig<64, 64, 2, 6, BF16>{});
      if (chunk == 128) return run(FaFwdConfig<64, 128, 2, 4, BF16>{});
      return run(FaFwdConfig<64, 256, 1, 3, BF16>{});
    case 128:
      if (chunk == 64) return run(FaFwdConfig<128, 64, 2, 4, BF16>{});
      if (chunk == 128) return run(FaFwdConfig<128, 128, 2, 4, BF16>{});
      return run(FaFwdConfig<128, 256, 1, 3, BF16>{});
    case 256:
      if (chunk == 64) return run(FaFwdConfig<256, 64, 1, 2, BF16>{});
      if (chunk == 128) return run(FaFwdConfig<256, 128, 1, 2, BF16>{});
      return run(FaFwdConfig<256, 256, 1, 2, BF16>{});
    default:
      return fail(kErrUnsupported, "fa_fwd: dqk=%d not built into libattn_b200 (64, 128, 256)", dqk);
  }
}

int fa_fwd_common(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Lq, int Lkv,
                  int dqk, int dv, int dtype, float scale, int causal, void* stream, bool profile, float* ms) {
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "fa_fwd: B and H must be positive");
  if (dtype != ATTN_B200_F16 && dtype != ATTN_B200_BF16) return fail(kErrInvalidArgument, "fa_fwd: dtype %d", dtype);
  FaFwdArgs a{q, k, v, o, lse, B * H, Lq, Lkv, dv, scale, causal};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dtype == ATTN_B200_BF16 ? fa_fwd_dispatch<true>(a, dqk, st, profile, ms)
                                 : fa_fwd_dispatch<false>(a, dqk, st, profile, ms);
}

int fa_bwd_common(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse, void* dq,
                  void* dk, void* dv, int B, int H, int Lq, int Lkv, int d, int dtype, float scale, int causal, void* stream,
                  bool profile, float* ms) {
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "fa_bwd: B and H must be positive");
  if (dtype != ATTN_B200_F16 && dtype != ATTN_B200_BF16) return fail(kErrInvalidArgument, "fa_bwd: dtype %d", dtype);
  FaBwdArgs a{q, k, v, o, dout, lse, dq, dk, dv, B * H, Lq, Lkv, d, scale, causal};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto run = [&](auto d_tag, auto bf16_tag) -> int {
    constexpr int D = decltype(d_tag)::value;
    constexpr bool BF16 = decltype(bf16_tag)::value;
    if (!profile) return fa_bwd_launch<D, BF16>(a, st);
    *ms = profile_loop([&] { return fa_bwd_launch<D, BF16>(a, st); }, st);
    return *ms < 0.f ? kErrCuda : kOk;
  };
  const bool bf16 = dtype == ATTN_B200_BF16;
  if (d == 64) return bf16 ? run(std::integral_constant<int, 64>{}, std::true_type{}) : run(std::integral_constant<int, 64>{}, std::false_type{});
  if (d == 128) return bf16 ? run(std::integral_constant<int, 128>{}, std::true_type{}) : run(std::integral_constant<int, 128>{}, std::false_type{});
  return fail(kErrUnsupported, "fa_bwd: head dimension %d (q, k and v must share 64 or 128)", d);
}

// RetNet head-dim pairs built into this library (others: per-config libraries from the tuner).
constexpr int chunk_of(int d) { return d % 256 == 0 ? 256 : d % 128 == 0 ? 128 : 64; }
// CTA pairs (cta_group::2, 256-row tiles) wherever the output chunks are wide enough to be split between two CTAs
constexpr bool pair_of(int chunk_a, int chunk_b) { return chunk_a >= 128 && chunk_b >= 128; }

template <bool BF16, bool BWD>
int ret_dispatch(const RetArgs& a, cudaStream_t st) {
#define AB200_RET_CASE(DQK, DV)                                                                        \
  if (a.dqk == DQK && a.dv == DV) {                                                                    \
    if constexpr (BWD)                                                                                 \
      return ret_bwd_launch<DQK, DV, chunk_of(DV), chunk_of(DQK), BF16, pair_of(chunk_of(DV), chunk_of(DQK))>(a, st); \
    else return ret_fwd_launch<DQK, chunk_of(DV), BF16, pair_of(chunk_of(DV), 128)>(a, st);              \
  }
  AB200_RET_CASE(64, 64)
  AB200_RET_CASE(64, 128)
  AB200_RET_CASE(128, 128)
  AB200_RET_CASE(128, 256)
  AB200_RET_CASE(256, 256)
  AB200_RET_CASE(256, 512)
#undef AB200_RET_CASE
  return fail(kErrUnsupported, "retnet: (dqk, dv) = (%d, %d) not built into libattn_b200", a.dqk, a.dv);
}

int ret_common(bool bwd, const RetArgs& a, int dtype, void* stream, bool profile, float* ms) {
  if (dtype != ATTN_B200_F16 && dtype != ATTN_B200_BF16) return fail(kErrInvalidArgument, "retnet: dtype %d", dtype);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  auto once = [&]() -> int {
    if (dtype == ATTN_B200_BF16) return bwd ? ret_dispatch<true, true>(a, st) : ret_dispatch<true, false>(a, st);
    return bwd ? ret_dispatch<false, true>(a, st) : ret_dispatch<false, false>(a, st);
  };
  if (!profile) return once();
  *ms = profile_loop(once, st);
  return *ms < 0.f ? kErrCuda : kOk;
}

RetArgs ret_args(const void* q, const void* k, const void* v, const void* mask, const float* decay, void* o, float* r,
                 const void* dout, void* dq, void* dk, void* dv_out, int B, int H, int Lq, int Lkv, int dqk, int dv,
                 float scale, int causal, void* workspace = nullptr, size_t workspace_bytes = 0) {
  RetArgs a{};
  a.workspace = workspace;
  a.workspace_bytes = workspace_bytes;
  a.q = q; a.k = k; a.v = v; a.mask = mask; a.decay = decay; a.o = o; a.r = r;
  a.dout = dout; a.dq = dq; a.dk = dk; a.dv_out = dv_out;
  a.BH = B * H; a.H = H; a.Lq = Lq; a.Lkv = Lkv; a.dqk = dqk; a.dv = dv; a.scale = scale; a.causal = causal;
  return a;
}

}  // namespace

extern "C" {

const char* attn_b200_last_error(void) { return error_buffer(); }

int attn_b200_device_status(int clear) {
  int det = 0;
  return read_device_status(clear, &det);
}

int attn_b200_abi_version(void) { return 1; }

int attn_b200_fa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Lq,
                     int Lkv, int dqk, int dv, int dtype, float scale, int causal, void* stream) {
  return fa_fwd_common(q, k, v, o, lse, B, H, Lq, Lkv, dqk, dv, dtype, scale, causal, stream, false, nullptr);
}

float attn_b200_fa_fwd_profile(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                               int Lq, int Lkv, int dqk, int dv, int dtype, float scale, int causal,
                               void* stream) {
  float ms = -1.f;
  int rc = fa_fwd_common(q, k, v, o, lse, B, H, Lq, Lkv, dqk, dv, dtype, scale, causal, stream, true, &ms);
  return rc == kOk ? ms : -1.f;
}

int attn_b200_fa_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                     void* dq, void* dk, void* dv, int B, int H, int Lq, int Lkv, int d, int dtype, float scale,
                     int causal, void* stream) {
  return fa_bwd_common(q, k, v, o, dout, lse, dq, dk, dv, B, H, Lq, Lkv, d, dtype, scale, causal, stream, false, nullptr);
}

float attn_b200_fa_bwd_profile(const void* q, const void* k, const void* v, const void* o, const void* dout,
                               const float* lse, void* dq, void* dk, void* dv, int B, int H, int Lq, int Lkv, int d,
                               int dtype, float scale, int causal, void* stream) {
  float ms = -1.f;
  int rc = fa_bwd_common(q, k, v, o, dout, lse, dq, dk, dv, B, H, Lq, Lkv, d, dtype, scale, causal, stream, true, &ms);
  return rc == kOk ? ms : -1.f;
}

int attn_b200_ret_fwd(const void* q, const void* k, const void* v, const void* mask, void* o, float* r, int B, int H,
                      int Lq, int Lkv, int dqk, int dv, int dtype, float scale, const float* decay, int causal,
                      void* stream) {
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "ret_fwd: B and H must be positive");
  return ret_common(false, ret_args(q, k, v, mask, decay, o, r, nullptr, nullptr, nullptr, nullptr, B, H, Lq, Lkv, dqk,
                                    dv, scale, causal), dtype, stream, false, nullptr);
}

float attn_b200_ret_fwd_profile(const void* q, const void* k, const void* v, const void* mask, void* o, float* r, int B,
                                int H, int Lq, int Lkv, int dqk, int dv, int dtype, float scale, const float* decay,
                                int causal, void* stream) {
  float ms = -1.f;
  if (B <= 0 || H <= 0) return -1.f;
  int rc = ret_common(false, ret_args(q, k, v, mask, decay, o, r, nullptr, nullptr, nullptr, nullptr, B, H, Lq, Lkv,
                                      dqk, dv, scale, causal), dtype, stream, true, &ms);
  return rc == kOk ? ms : -1.f;
}

// Size of the reference's dq_accum tensor (fp32 [B, H, Lq, dqk]): what a caller of the reference's ABI hands over.
static size_t dq_accum_bytes(const void* dq_accum, int B, int H, int Lq, int dqk) {
  if (dq_accum == nullptr || B <= 0 || H <= 0 || Lq <= 0 || dqk <= 0) return 0;
  return static_cast<size_t>(B) * H * Lq * dqk * sizeof(float);
}

int attn_b200_ret_bwd_ws(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r,
                         void* dq, void* dk, void* dv_out, void* workspace, size_t workspace_bytes, int B, int H, int Lq,
                         int Lkv, int dqk, int dv, int dtype, float scale, const float* decay, int causal, void* stream) {
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "ret_bwd: B and H must be positive");
  return ret_common(true, ret_args(q, k, v, mask, decay, nullptr, const_cast<float*>(r), dout, dq, dk, dv_out, B, H, Lq,
                                   Lkv, dqk, dv, scale, causal, workspace, workspace_bytes), dtype, stream, false, nullptr);
}

size_t attn_b200_ret_bwd_workspace_bytes(int H, int Lq, int Lkv) {
  if (H <= 0 || Lq <= 0 || Lkv <= 0) return 0;
  return static_cast<size_t>(H) * Lq * Lkv * 2u;
}

int attn_b200_ret_bwd(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r,
                      void* dq, void* dk, void* dv_out, float* dq_accum, int B, int H, int Lq, int Lkv, int dqk, int dv,
                      int dtype, float scale, const float* decay, int causal, void* stream) {
  // dq_accum is scratch in the reference's ABI (fp32 [B, H, Lq, dqk], python/ops/retnet_interface.py:48-54); here it
  // is scratch too: room for a transposed copy of the mask when it is large enough, unused otherwise
  return attn_b200_ret_bwd_ws(q, k, v, mask, dout, r, dq, dk, dv_out, dq_accum, dq_accum_bytes(dq_accum, B, H, Lq, dqk), B, H,
                              Lq, Lkv, dqk, dv, dtype, scale, decay, causal, stream);
}

float attn_b200_ret_bwd_profile(const void* q, const void* k, const void* v, const void* mask, const void* dout,
                                const float* r, void* dq, void* dk, void* dv_out, float* dq_accum, int B, int H, int Lq,
                                int Lkv, int dqk, int dv, int dtype, float scale, const float* decay, int causal,
                                void* stream) {
  float ms = -1.f;
  if (B <= 0 || H <= 0) return -1.f;
  int rc = ret_common(true, ret_args(q, k, v, mask, decay, nullptr, const_cast<float*>(r), dout, dq, dk, dv_out, B, H,
                                     Lq, Lkv, dqk, dv, scale, causal, dq_accum, dq_accum_bytes(dq_accum, B, H, Lq, dqk)),
                      dtype, stream, true, &ms);
  return rc == kOk ? ms : -1.f;
}

size_t attn_b200_ret_bwd_noalloc_max_bytes(void) { return kNoAllocScratchBytes; }

int attn_b200_ret_bwd_noalloc(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r,
                              void* dq, void* dk, void* dv_out, int B, int H, int Lq, int Lkv, int dqk, int dv, int dtype,
                              float scale, const float* decay, int causal, void* stream) {
  if (B <= 0 || H <= 0 || Lq <= 0 || Lkv <= 0) return fail(kErrInvalidArgument, "ret_bwd_noalloc: sizes must be positive");
  // the only scratch the backward uses is the transposed copy of a mask tensor; it has to fit the library's own array
  const size_t need = mask != nullptr ? static_cast<size_t>(H) * Lq * Lkv * 2u : 0;
  if (need > kNoAllocScratchBytes)
    return fail(kErrInvalidArgument,
                "ret_bwd_noalloc: the mask needs %zu bytes of scratch (H * Lq * Lkv * 2) but this entry point holds %zu "
                "(H * Lq * Lkv <= %zu); call attn_b200_ret_bwd_ws with a workspace of your own for larger masks",
                need, kNoAllocScratchBytes, kNoAllocScratchBytes / 2);
  void* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  NoAllocScope no_alloc;  // nothing below may allocate: no pinned status mirror, no cudaFree(nullptr)
  return ret_common(true, ret_args(q, k, v, mask, decay, nullptr, const_cast<float*>(r), dout, dq, dk, dv_out, B, H, Lq,
                                   Lkv, dqk, dv, scale, causal, scratch, kNoAllocScratchBytes), dtype, stream, false, nullptr);
}

int attn_b200_ret_chunk_fwd(const void* q, const void* k, const void* v, const float* decay, void* o, int B, int H, int L,
                            int dqk, int dv, int dtype, float scale, void* stream) {
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "ret_chunk_fwd: B and H must be positive");
  if (dtype != ATTN_B200_F16 && dtype != ATTN_B200_BF16) return fail(kErrInvalidArgument, "ret_chunk_fwd: dtype %d", dtype);
  RetChunkArgs a{q, k, v, decay, o, B * H, H, L, dqk, dv, scale};
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dtype == ATTN_B200_BF16 ? ret_chunk_dispatch<true>(a, st) : ret_chunk_dispatch<false>(a, st);
}

size_t attn_b200_ret_chunk_workspace_bytes(int B, int H, int L, int dqk, int dv, int segments) {
  if (B <= 0 || H <= 0 || L <= 0 || dqk <= 0 || dv <= 0 || segments < 0) return 0;
  const int g = segments > 0 ? segments : ret_chunk_preferred_segments(B * H, L, dv);
  return ret_chunk_workspace_bytes(B * H, L, dqk, dv, g);
}

int attn_b200_ret_chunk_fwd_ws(const void* q, const void* k, const void* v, const float* decay, void* o, void* workspace,
                               size_t workspace_bytes, int segments, int B, int H, int L, int dqk, int dv, int dtype, float scale,
                               void* stream) {
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "ret_chunk_fwd: B and H must be positive");
  if (dtype != ATTN_B200_F16 && dtype != ATTN_B200_BF16) return fail(kErrInvalidArgument, "ret_chunk_fwd: dtype %d", dtype);
  RetChunkArgs a{q, k, v, decay, o, B * H, H, L, dqk, dv, scale};
  a.workspace = workspace;
  a.workspace_bytes = workspace ? workspace_bytes : 0;
  a.segments = segments;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return dtype == ATTN_B200_BF16 ? ret_chunk_dispatch<true>(a, st) : ret_chunk_dispatch<false>(a, st);
}

int attn_b200_selftest_gemm_ss(const void* a, const void* b, float* d, int N, int K, int dtype, void* stream) {
  return selftest_gemm_ss(a, b, d, N, K, dtype, reinterpret_cast<cudaStream_t>(stream));
}
int attn_b200_selftest_gemm_ts(const void* p, const void* v, float* d, int N, int dtype, void* stream) {
  return selftest_gemm_ts(p, v, d, N, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int attn_b200_selftest_pair(const void* a, const void* b, const void* t, float* z, float* d, int K, int N2, int dtype,
                            void* stream) {
  return selftest_pair(a, b, t, z, d, K, N2, dtype, reinterpret_cast<cudaStream_t>(stream));
}

int attn_b200_selftest_wait(int limit_us, int whole_warp, void* stream) {
  return selftest_wait(limit_us, whole_warp, reinterpret_cast<cudaStream_t>(stream));
}

}  // extern "C"
