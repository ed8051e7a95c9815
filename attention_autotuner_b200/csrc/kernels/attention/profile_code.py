"""Launch-shim source of one flash-attention tile configuration, filled by
``str.format_map(config.substitution_map())``. Same role and the same two legacy symbols as the
reference's csrc/kernels/attention/regfuse/profile_code.py:
    extern "C" int   kernel_entry(half* q, half* k, half* v, half* o, int B, int H, int Seq_k, int Seq_q)
    extern "C" float profile     (half* q, half* k, half* v, half* o, int B, int H, int Seq_q, int Seq_k)
(fixed 0.125 softmax scale, non-causal, default stream, as in the reference), plus *_ex variants that
take scale, causal flag, LSE pointer and stream."""

global_vars = """
#include "fa_fwd_launch.cuh"
using namespace ab200;
using Cfg = {cfg_type};
constexpr int kDv = {D};
static int run(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Seq_k, int Seq_q,
               float scale, int causal, void* stream) {{
  if (B <= 0 || H <= 0) return fail(kErrInvalidArgument, "B and H must be positive");
  FaFwdArgs a{{q, k, v, o, lse, B * H, Seq_q, Seq_k, kDv, scale, causal}};
  return {launcher}<Cfg>(a, reinterpret_cast<cudaStream_t>(stream));
}}
extern "C" const char* last_error() {{ return error_buffer(); }}
extern "C" int device_status(int clear) {{ int det = 0; return read_device_status(clear, &det); }}
"""

profile_func = """
extern "C" float profile_ex(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Seq_q,
                            int Seq_k, float scale, int causal, void* stream) {{
  return profile_loop([&] {{ return run(q, k, v, o, lse, B, H, Seq_k, Seq_q, scale, causal, stream); }},
                      reinterpret_cast<cudaStream_t>(stream));
}}
extern "C" float profile(void* q, void* k, void* v, void* o, int B, int H, int Seq_q, int Seq_k) {{
  return profile_ex(q, k, v, o, nullptr, B, H, Seq_q, Seq_k, 0.125f, 0, nullptr);
}}
"""

kernel_entry = """
extern "C" int kernel_entry_ex(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                               int Seq_k, int Seq_q, float scale, int causal, void* stream) {{
  return run(q, k, v, o, lse, B, H, Seq_k, Seq_q, scale, causal, stream);
}}
extern "C" int kernel_entry(void* q, void* k, void* v, void* o, int B, int H, int Seq_k, int Seq_q) {{
  return run(q, k, v, o, nullptr, B, H, Seq_k, Seq_q, 0.125f, 0, nullptr);
}}
"""

profile_code = global_vars + profile_func
kernel_code = global_vars + kernel_entry + profile_func
