/*
 * C ABI of libattn_b200.so: fused attention / RetNet kernels for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; every tensor pointer is a DEVICE pointer owned by the caller, dense and
 * row-major in the layouts given below, 16-byte aligned. The library allocates no device memory.
 * Kernels are launched asynchronously on `stream` (a cudaStream_t passed as void*, NULL = default
 * stream). Every function returns 0 on success and one of ATTN_B200_ERR_* otherwise; the text of the
 * last error of the calling thread is available from attn_b200_last_error().
 *
 * The reference project binds, through ctypes, two symbols of each library it compiles
 * (python/autotuner/runtime.py:79-82 and python/autotuner/base_tunner.py:101-105):
 *     int   kernel_entry(ptrs..., int B, int H, int Seq_k, int Seq_q);
 *     float profile     (ptrs..., int B, int H, int Seq_q, int Seq_k);
 * The per-configuration libraries built by attention_autotuner_b200.autotuner keep exactly those two
 * symbols (second half of this header). libattn_b200.so itself exports the general entry points
 * below, which take the head dimensions, dtype, scale and stream explicitly.
 */
#ifndef ATTN_B200_H_
#define ATTN_B200_H_

#ifdef __cplusplus
extern "C" {
#endif

#define ATTN_B200_OK 0
#define ATTN_B200_ERR_INVALID_ARGUMENT 1 /* null / misaligned pointer, non-positive size, bad dtype   */
#define ATTN_B200_ERR_UNSUPPORTED 2      /* head dims or tile config not built into the library        */
#define ATTN_B200_ERR_CUDA 3             /* a CUDA call failed; see attn_b200_last_error()              */
#define ATTN_B200_ERR_DEVICE 4           /* a kernel gave up on a bounded wait; results are invalid    */

#define ATTN_B200_F16 0
#define ATTN_B200_BF16 1

/* Text of the calling thread's most recent error ("" if none). Never NULL. */
const char* attn_b200_last_error(void);

/* Synchronises the current device and returns the sticky device status word written by the kernels
 * (0 = ok, 1 = a bounded barrier wait expired). `clear` != 0 resets it. Returns -1 if the read failed. */
int attn_b200_device_status(int clear);

/* ABI version of this header (bumped on incompatible changes). */
int attn_b200_abi_version(void);

/*
 * Flash-attention forward:  O = softmax(Q K^T * scale  [causal]) V,  optional LSE.
 * Replaces the path python/ops/attention_interface.py:11-35 -> Runtime.apply
 * (python/autotuner/runtime.py:74-82) -> kernel_entry -> flashattn_fwd_regfuse / flashattn_fwd_smemfuse
 * (csrc/kernels/attention/regfuse/regfuse.h:48, csrc/kernels/attention/smemfuse/smemfuse.h:61).
 *   q [B,H,Lq,dqk]  k [B,H,Lkv,dqk]  v [B,H,Lkv,dv]  o [B,H,Lq,dv]  (dtype)   lse [B,H,Lq] fp32 or NULL
 *   dqk in {64,128,256}, dv in {64,128,256,512}; dtype ATTN_B200_F16 / ATTN_B200_BF16.
 *   scale > 0 (the reference hard-codes 0.125). causal != 0 masks key j for query i when
 *   j > i + (Lkv - Lq). Lq, Lkv need not be multiples of the tile size.
 */
int attn_b200_fa_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H, int Lq,
                     int Lkv, int dqk, int dv, int dtype, float scale, int causal, void* stream);

/* Same arguments; runs one warm-up launch and then about 100 ms of launches between two CUDA events
 * on `stream`, as the reference's generated profile() does
 * (csrc/kernels/attention/regfuse/profile_code.py:28-63). Returns ms per launch, or -1 on error. */
float attn_b200_fa_fwd_profile(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                               int Lq, int Lkv, int dqk, int dv, int dtype, float scale, int causal,
                               void* stream);

/*
 * Flash-attention backward:  dQ, dK, dV of the forward above, given its output o, its log-sum-exp lse and dO.
 * The reference declares this backward and leaves it empty (python/ops/attention_interface.py:38-39); this entry
 * point is what that method would bind. Three kernels (dV, dK, dQ), each owning its output tile: no atomics and no
 * workspace; P is recomputed from lse, delta = rowsum(dO .* O) is computed inside the kernels.
 *   q, o, dout, dq [B,H,Lq,d]   k, v, dk, dv [B,H,Lkv,d]   (dtype)    lse [B,H,Lq] fp32 (from attn_b200_fa_fwd)
 *   d in {64,128} for q, k and v alike. causal != 0 needs Lq == Lkv. scale as given to the forward.
 */
int attn_b200_fa_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                     void* dq, void* dk, void* dv, int B, int H, int Lq, int Lkv, int d, int dtype, float scale,
                     int causal, void* stream);

/* Same arguments; timing loop as attn_b200_fa_fwd_profile. Returns ms per backward (three launches), or -1. */
float attn_b200_fa_bwd_profile(const void* q, const void* k, const void* v, const void* o, const void* dout,
                               const float* lse, void* dq, void* dk, void* dv, int B, int H, int Lq, int Lkv, int d,
                               int dtype, float scale, int causal, void* stream);

/*
 * RetNet parallel forward:  S~ = (Q K^T * scale) .* M,  r = max(sum_j |S~|, 1),  O = (S~ / r) V.
 * Replaces python/ops/retnet_interface.py:11-33 -> Runtime.apply -> kernel_entry -> ret_fwd_regfuse /
 * ret_fwd_smemfuse (csrc/kernels/retnet/regfuse/regfuse.h:47, csrc/kernels/retnet/smemfuse/smemfuse.h:62).
 *   q [B,H,Lq,dqk]  k [B,H,Lkv,dqk]  v [B,H,Lkv,dv]  o [B,H,Lq,dv] (dtype)   r [B,H,Lq] fp32 (output)
 *   The mask M is given in exactly one of two forms:
 *     mask  != NULL, decay == NULL : the reference's general tensor [H,Lq,Lkv] (dtype), broadcast over batch;
 *                                    needs Lkv % 8 == 0. causal != 0 declares it lower triangular
 *                                    (M[i,j] = 0 for j > i) so that blocks above the diagonal are skipped.
 *     mask  == NULL, decay != NULL : per-head decay, decay = device pointer to H floats gamma_h,
 *                                    M[h,i,j] = gamma_h^(i-j) for i >= j and 0 otherwise; built in registers.
 *   scale: the reference has none (= 1.0). (dqk, dv) in {(64,64),(64,128),(128,128),(128,256),(256,256),(256,512)}.
 */
int attn_b200_ret_fwd(const void* q, const void* k, const void* v, const void* mask, void* o, float* r, int B, int H,
                      int Lq, int Lkv, int dqk, int dv, int dtype, float scale, const float* decay, int causal,
                      void* stream);
float attn_b200_ret_fwd_profile(const void* q, const void* k, const void* v, const void* mask, void* o, float* r, int B,
                                int H, int Lq, int Lkv, int dqk, int dv, int dtype, float scale, const float* decay,
                                int causal, void* stream);

/*
 * RetNet parallel backward (r is a constant, no gradient for the mask):
 *   P = S~ / r,  dV = P^T dO,  G = ((dO V^T) / r) .* M * scale,  dK = G^T Q,  dQ = G K.
 * Replaces python/ops/retnet_interface.py:36-55 -> kernel_entry -> ret_bwd_colblock + convert_dq
 * (csrc/kernels/retnet/bwd/bwd_colblock.h:81, 742). Tensor order follows the reference's
 * [q,k,v,mask,do,r,dq,dk,dv,dq_accum]; dq_accum (fp32 [B,H,Lq,dqk] in the reference) is accepted and
 * ignored, may be NULL: every output tile is owned by one CTA, nothing is accumulated with atomics.
 *   dout [B,H,Lq,dv]  r [B,H,Lq] (from the forward)  dq [B,H,Lq,dqk]  dk [B,H,Lkv,dqk]  dv_out [B,H,Lkv,dv]
 * Outputs are fully overwritten.
 */
int attn_b200_ret_bwd(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r,
                      void* dq, void* dk, void* dv_out, float* dq_accum, int B, int H, int Lq, int Lkv, int dqk, int dv,
                      int dtype, float scale, const float* decay, int causal, void* stream);
float attn_b200_ret_bwd_profile(const void* q, const void* k, const void* v, const void* mask, const void* dout,
                                const float* r, void* dq, void* dk, void* dv_out, float* dq_accum, int B, int H, int Lq,
                                int Lkv, int dqk, int dv, int dtype, float scale, const float* decay, int causal,
                                void* stream);

/*
 * Building-block self tests (single CTA, used by the test-suite to pin the tcgen05 / TMA descriptors):
 *   ss: d[128,N] = a[128,K] * b[N,K]^T       K in {64,128,192,256}, N multiple of 32, N*K <= 32768
 *   ts: d[128,N] = p[128,128] * v[128,N]     N in {64,128,192,256}
 * a, b, p, v are 16-bit (dtype), d is fp32. No counterpart in the reference.
 */
int attn_b200_selftest_gemm_ss(const void* a, const void* b, float* d, int N, int K, int dtype, void* stream);
int attn_b200_selftest_gemm_ts(const void* p, const void* v, float* d, int N, int dtype, void* stream);

/*
 * CTA-pair building block (one cluster of two CTAs, tcgen05 cta_group::2), the RetNet chain in miniature:
 *   z[256,128] = a[256,K] * b[128,K]^T     K in {64,128,192,256}
 *   d[256,N2]  = w[256,128] * t[128,N2]    w = 16-bit copy of z kept in tensor memory, N2 in {128,256}
 * a, b, t are 16-bit (dtype), z and d fp32. No counterpart in the reference.
 */
int attn_b200_selftest_pair(const void* a, const void* b, const void* t, float* z, float* d, int K, int N2, int dtype,
                            void* stream);

#ifdef __cplusplus
}
#endif

#endif /* ATTN_B200_H_ */
