"""Launch-shim source of one RetNet-forward tile configuration (filled by str.format_map). Keeps the two
symbols the reference binds (csrc/kernels/retnet/regfuse/profile_code.py:30,72):
    extern "C" int   kernel_entry(half* q, half* k, half* v, half* mask, half* o, float* r, int B, int H, int Seq_k, int Seq_q)
    extern "C" float profile     (half* q, half* k, half* v, half* mask, half* o, float* r, int B, int H, int Seq_q, int Seq_k)
(no score scale, general mask, default stream, as in the reference) plus *_ex variants taking scale, a
per-head decay pointer (mask may then be NULL), the lower-triangular hint and the stream."""

global_vars = """
#include "chain_launch.cuh"
using namespace ab200;
static int run(const void* q, const void* k, const void* v, const void* mask, void* o, float* r, int B, int H, int Seq_k,
               int Seq_q, float scale, const float* decay, int causal, void* stream) {{
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "B and H must be positive");
  RetArgs a{{}};
  a.q = q; a.k = k; a.v = v; a.mask = mask; a.decay = decay; a.o = o; a.r = r;
  a.BH = B * H; a.H = H; a.Lq = Seq_q; a.Lkv = Seq_k; a.dqk = {Kd}; a.dv = {D}; a.scale = scale; a.causal = causal;
  return ret_fwd_launch<{Kd}, {dv_chunk}, {bf16}, {cta_pair_bool}>(a, reinterpret_cast<cudaStream_t>(stream));
}}
extern "C" const char* last_error() {{ return error_buffer(); }}
extern "C" int device_status(int clear) {{ int det = 0; return read_device_status(clear, &det); }}
"""

profile_func = """
extern "C" float profile_ex(const void* q, const void* k, const void* v, const void* mask, void* o, float* r, int B, int H,
                            int Seq_q, int Seq_k, float scale, const float* decay, int causal, void* stream) {{
  return profile_loop([&] {{ return run(q, k, v, mask, o, r, B, H, Seq_k, Seq_q, scale, decay, causal, stream); }},
                      reinterpret_cast<cudaStream_t>(stream));
}}
extern "C" float profile(void* q, void* k, void* v, void* mask, void* o, float* r, int B, int H, int Seq_q, int Seq_k) {{
  return profile_ex(q, k, v, mask, o, r, B, H, Seq_q, Seq_k, 1.0f, nullptr, 0, nullptr);
}}
"""

kernel_entry = """
extern "C" int kernel_entry_ex(const void* q, const void* k, const void* v, const void* mask, void* o, float* r, int B,
                               int H, int Seq_k, int Seq_q, float scale, const float* decay, int causal, void* stream) {{
  return run(q, k, v, mask, o, r, B, H, Seq_k, Seq_q, scale, decay, causal, stream);
}}
extern "C" int kernel_entry(void* q, void* k, void* v, void* mask, void* o, float* r, int B, int H, int Seq_k, int Seq_q) {{
  return run(q, k, v, mask, o, r, B, H, Seq_k, Seq_q, 1.0f, nullptr, 0, nullptr);
}}
"""

profile_code = global_vars + profile_func
kernel_code = global_vars + kernel_entry + profile_func
