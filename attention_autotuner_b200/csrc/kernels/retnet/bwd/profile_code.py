"""Launch-shim source of one RetNet-backward tile configuration (filled by str.format_map). Keeps the two
symbols the reference binds (csrc/kernels/retnet/bwd/profile_code.py:50,98), with its tensor order
q, k, v, mask, do, r, dq, dk, dv, dqaccum, plus *_ex variants. dqaccum is scratch, as in the reference: with a mask
tensor the backward puts a transposed copy of the mask there when it is large enough (the legacy symbols assume the
reference's fp32 [B, H, Seq_q, Kd] tensor; the *_ex symbols take its size in bytes)."""

global_vars = """
#include "chain_launch.cuh"
using namespace ab200;
static int run(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r, void* dq,
               void* dk, void* dv, float* dqaccum, int B, int H, int Seq_k, int Seq_q, float scale, const float* decay,
               int causal, void* stream, size_t dqaccum_bytes) {{
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "B and H must be positive");
  RetArgs a{{}};
  a.workspace = dqaccum;
  a.workspace_bytes = dqaccum ? dqaccum_bytes : 0;
  a.q = q; a.k = k; a.v = v; a.mask = mask; a.decay = decay; a.r = const_cast<float*>(r);
  a.dout = dout; a.dq = dq; a.dk = dk; a.dv_out = dv;
  a.BH = B * H; a.H = H; a.Lq = Seq_q; a.Lkv = Seq_k; a.dqk = {Kd}; a.dv = {D}; a.scale = scale; a.causal = causal;
  return ret_bwd_launch<{Kd}, {D}, {dv_chunk}, {dq_chunk}, {bf16}, {cta_pair_bool}>(a, reinterpret_cast<cudaStream_t>(stream));
}}
// size of the reference's dq_accum tensor: fp32 [B, H, Seq_q, Kd]
static size_t reference_dqaccum_bytes(int B, int H, int Seq_q) {{
  return (B > 0 && H > 0 && Seq_q > 0) ? static_cast<size_t>(B) * H * Seq_q * {Kd} * sizeof(float) : 0;
}}
extern "C" const char* last_error() {{ return error_buffer(); }}
extern "C" int device_status(int clear) {{ int det = 0; return read_device_status(clear, &det); }}
"""

profile_func = """
extern "C" float profile_ex(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r,
                            void* dq, void* dk, void* dv, float* dqaccum, int B, int H, int Seq_q, int Seq_k, float scale,
                            const float* decay, int causal, void* stream, size_t dqaccum_bytes) {{
  return profile_loop([&] {{ return run(q, k, v, mask, dout, r, dq, dk, dv, dqaccum, B, H, Seq_k, Seq_q, scale, decay,
                                        causal, stream, dqaccum_bytes); }}, reinterpret_cast<cudaStream_t>(stream));
}}
extern "C" float profile(void* q, void* k, void* v, void* mask, void* dout, float* r, void* dq, void* dk, void* dv,
                         float* dqaccum, int B, int H, int Seq_q, int Seq_k) {{
  return profile_ex(q, k, v, mask, dout, r, dq, dk, dv, dqaccum, B, H, Seq_q, Seq_k, 1.0f, nullptr, 0, nullptr,
                    reference_dqaccum_bytes(B, H, Seq_q));
}}
"""

kernel_entry = """
extern "C" int kernel_entry_ex(const void* q, const void* k, const void* v, const void* mask, const void* dout,
                               const float* r, void* dq, void* dk, void* dv, float* dqaccum, int B, int H, int Seq_k,
                               int Seq_q, float scale, const float* decay, int causal, void* stream, size_t dqaccum_bytes) {{
  return run(q, k, v, mask, dout, r, dq, dk, dv, dqaccum, B, H, Seq_k, Seq_q, scale, decay, causal, stream, dqaccum_bytes);
}}
extern "C" int kernel_entry(void* q, void* k, void* v, void* mask, void* dout, float* r, void* dq, void* dk, void* dv,
                            float* dqaccum, int B, int H, int Seq_k, int Seq_q) {{
  return run(q, k, v, mask, dout, r, dq, dk, dv, dqaccum, B, H, Seq_k, Seq_q, 1.0f, nullptr, 0, nullptr,
             reference_dqaccum_bytes(B, H, Seq_q));
}}
"""

profile_code = global_vars + profile_func
kernel_code = global_vars + kernel_entry + profile_func
