/*
 * C ABI of libattn_b200.so: fused attention / RetNet kernels for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; every tensor pointer is a DEVICE pointer owned by the caller, dense and
 * row-major in the layouts given below. Alignment: inputs of the forward entry points (q, k, v, mask) 16 bytes,
 * every 16-bit OUTPUT tensor (o, dq, dk, dv) 32 bytes (they are written with 256-bit stores), and all eight 16-bit
 * tensors of attn_b200_fa_bwd 32 bytes; fp32 vectors (lse, r, decay) 4 bytes. A misaligned pointer is rejected with
 * ATTN_B200_ERR_INVALID_ARGUMENT. The library allocates no device memory (on its first launch per device it pins two
 * ints of host memory for the status word described at attn_b200_device_status).
 * Kernels are launched asynchronously on `stream` (a cudaStream_t passed as void*, NULL = default
 * stream). Every function returns 0 on success and one of ATTN_B200_ERR_* otherwise; the text of the
 * last error of the calling thread is available from attn_b200_last_error().
 *
 * The reference project binds, through ctypes, two symbols of each library it compiles
 * (python/autotuner/runtime.py:79-82 and python/autotuner/base_tunner.py:101-105):
 *     int   kernel_entry(ptrs..., int B, int H, int Seq_k, int Seq_q);
 *     float profile     (ptrs..., int B, int H, int Seq_q, int Seq_k);
 * The per-configuration libraries built by attention_autotuner_b200.autotuner keep exactly those two
 * symbols; their signatures, which differ per operation, are given as function-pointer types in the second
 * half of this header. libattn_b200.so itself exports the general entry points below, which take the head
 * dimensions, dtype, scale and stream explicitly.
 */
#ifndef ATTN_B200_H_
#define ATTN_B200_H_

#include <stddef.h>

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
 * (0 = ok, 1 = a bounded barrier wait expired). `clear` != 0 resets it. Returns -1 if the read failed.
 * While the word is set, every launching entry point returns ATTN_B200_ERR_DEVICE without launching (it reads a
 * host-mapped copy of the word, no synchronisation), so a kernel that gave up cannot silently poison later results:
 * read and clear the status, then launch again. */
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
 * point is what that method would bind. Every output tile is owned by one CTA: no atomics and no workspace; P is
 * recomputed from lse. Three launches: a small kernel that computes delta = rowsum(dO .* O) and -lse / scale per
 * query, one kernel for dK and dV together, one for dQ. The per-query terms (16 bytes per query) are parked in the dq
 * buffer until the dQ kernel, which runs last, overwrites it: dq must not overlap any input, and ATTN_B200_FA_BWD_SPLIT=1
 * in the environment (or fewer than 16 queries) selects the older form with one kernel per gradient instead.
 *   q, o, dout, dq [B,H,Lq,d]   k, v, dk, dv [B,H,Lkv,d]   (dtype)    lse [B,H,Lq] fp32 (from attn_b200_fa_fwd)
 *   d in {64,128} for q, k and v alike. causal != 0 needs Lq == Lkv. scale as given to the forward.
 */
int attn_b200_fa_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                     void* dq, void* dk, void* dv, int B, int H, int Lq, int Lkv, int d, int dtype, float scale,
                     int causal, void* stream);

/* Same arguments; timing loop as attn_b200_fa_fwd_profile. Returns ms per backward (its three launches), or -1. */
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
 * [q,k,v,mask,do,r,dq,dk,dv,dq_accum]. Every output tile is owned by one CTA: nothing is accumulated with atomics.
 *   dout [B,H,Lq,dv]  r [B,H,Lq] (from the forward)  dq [B,H,Lq,dqk]  dk [B,H,Lkv,dqk]  dv_out [B,H,Lkv,dv]
 * Outputs are fully overwritten.
 *   dq_accum: scratch of the reference's shape (fp32 [B,H,Lq,dqk]) or NULL. The reference accumulates dQ in it; here it is
 *   scratch for something else: with a mask TENSOR, the kernels that own keys (dV, dK) need columns of M[h][query][key], and
 *   when dq_accum is given, holds at least H*Lq*Lkv 16-bit values (2*B*dqk >= Lkv) and Lq % 8 == 0, the mask is
 *   transposed into it once per call and read by rows; otherwise the columns are read and transposed in registers
 *   (same results, slower). Its contents are undefined after the call. Ignored with `decay`.
 */
int attn_b200_ret_bwd(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r,
                      void* dq, void* dk, void* dv_out, float* dq_accum, int B, int H, int Lq, int Lkv, int dqk, int dv,
                      int dtype, float scale, const float* decay, int causal, void* stream);
float attn_b200_ret_bwd_profile(const void* q, const void* k, const void* v, const void* mask, const void* dout,
                                const float* r, void* dq, void* dk, void* dv_out, float* dq_accum, int B, int H, int Lq,
                                int Lkv, int dqk, int dv, int dtype, float scale, const float* decay, int causal,
                                void* stream);

/* The same backward with the scratch given explicitly: `workspace` (device memory, 16-byte aligned, owned by the caller)
 * of `workspace_bytes` bytes; attn_b200_ret_bwd_workspace_bytes(H, Lq, Lkv) = H*Lq*Lkv*2 is what the transposed copy of
 * a mask tensor needs. NULL or too small: the slower in-register path. No counterpart in the reference (its scratch
 * is the dq_accum argument above). */
size_t attn_b200_ret_bwd_workspace_bytes(int H, int Lq, int Lkv);
int attn_b200_ret_bwd_ws(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r,
                         void* dq, void* dk, void* dv_out, void* workspace, size_t workspace_bytes, int B, int H, int Lq,
                         int Lkv, int dqk, int dv, int dtype, float scale, const float* decay, int causal, void* stream);

/*
 * The RetNet backward for callers that can neither bring scratch memory nor let the library allocate any. Such callers
 * exist wherever device memory is handed out by something other than cudaMalloc at call time: a serving process that
 * gave the whole HBM to its own pool at start-up and forbids allocations on the request path (an allocation there
 * synchronises the device and can fail under fragmentation), a plug-in running inside a host framework whose memory
 * budget it must not exceed, code on a latency-critical path where cudaMalloc's implicit synchronisation is not
 * acceptable. attn_b200_ret_bwd_ws wants a workspace from them and the Python operator allocates one; this entry
 * point does neither: the transposed copy of the mask goes into an array that is part of the library image itself.
 *   Same tensors and meaning as attn_b200_ret_bwd, without the dq_accum argument.
 *   Limit: the array has attn_b200_ret_bwd_noalloc_max_bytes() = 32 MiB, i.e. a mask tensor of at most H*Lq*Lkv = 16 Mi
 *   elements (8 heads x 1448 x 1448, 4 x 2048 x 2048, 16 x 1024 x 1024); a larger mask is rejected with
 *   ATTN_B200_ERR_INVALID_ARGUMENT and a message that names both sizes. With `decay` no scratch is used and there is no
 *   limit. Every device that loads the library holds the 32 MiB until the process exits.
 *   The call makes no cudaMalloc / cudaFree / cudaHostAlloc and calls no allocating library routine. The FIRST call on a
 *   device looks up the array's device address (cudaGetSymbolAddress, with that device current) and remembers it;
 *   make that first call before any stream capture begins on that device.
 *   The array is shared by all calls and keeps what the last call wrote; nothing in it has to start at zero (each
 *   call overwrites the part it reads), but two calls whose kernels overlap on the GPU (different streams, or threads
 *   without ordering between them) race on it: order them on one stream or with events.
 * No counterpart in the reference (its backward takes its scratch, dq_accum, from the caller).
 */
size_t attn_b200_ret_bwd_noalloc_max_bytes(void);
int attn_b200_ret_bwd_noalloc(const void* q, const void* k, const void* v, const void* mask, const void* dout, const float* r,
                              void* dq, void* dk, void* dv_out, int B, int H, int Lq, int Lkv, int dqk, int dv, int dtype,
                              float scale, const float* decay, int causal, void* stream);

/*
 * Chunkwise (recurrent-state) RetNet forward: the unnormalised retention
 *     O[i] = scale * sum_{j <= i} gamma_h^(i-j) (q_i . k_j) v_j
 * evaluated chunk by chunk with a running state, so the work grows with L instead of L^2. Replaces the reference's
 * retnet_recurrent_fwd (csrc/kernels/retnet/recurrent/recurrent.h:427-463: fp32 tensors laid out [bh, dim, L], a CUB
 * scan per (k, v) dimension pair, reached from benchmarks/retnet/retnet.cu:175-215) for a per-head constant decay, and
 * is the "chunkwise retnet" of its to-do list (README.md:103). Tensors use this library's layout and types:
 *   q, k [B,H,L,dqk]  v, o [B,H,L,dv]  (dtype)   decay: H floats gamma_h in (0, 1] (device)
 *   dqk in {128, 256}; dv a multiple of 64 up to 512. No normalisation, no r (that is the parallel form's).
 *   No scratch memory: every decay factor is applied in registers, in tensor memory or in place in shared memory.
 */
int attn_b200_ret_chunk_fwd(const void* q, const void* k, const void* v, const float* decay, void* o, int B, int H, int L,
                            int dqk, int dv, int dtype, float scale, void* stream);

/*
 * The same function with scratch memory, for few (batch, head) slices and long sequences, where a walk in order leaves
 * most SMs idle: the sequence is cut into segments; a first kernel computes the state every segment but the last leaves
 * behind on its own (fp32, one [dqk x dv] tile per slice and segment), then all segments run at once, each starting from
 * the decayed sum of the states before it. Same result as the walk in order up to rounding (the segment states are
 * exact fp32 sums of the same 16-bit products; the decay over a segment sits on the rows of K).
 *   segments = 0: the library chooses (as many as fill the SMs and the workspace holds; 1, the walk in order, when the
 *                 slices alone fill the GPU or workspace is null);  n > 0: min(n, chunks of 128) segments, an error
 *                 if the workspace is too small for them.
 *   attn_b200_ret_chunk_workspace_bytes: bytes for `segments` (0: for the library's choice; may be 0).
 * No counterpart in the reference (its recurrent kernel scans each (k, v) dimension pair over the whole sequence).
 */
size_t attn_b200_ret_chunk_workspace_bytes(int B, int H, int L, int dqk, int dv, int segments);
int attn_b200_ret_chunk_fwd_ws(const void* q, const void* k, const void* v, const float* decay, void* o, void* workspace,
                               size_t workspace_bytes, int segments, int B, int H, int L, int dqk, int dv, int dtype, float scale,
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

/*
 * The bounded wait in miniature: launches one warp that waits on a barrier nobody arrives at, with a limit of
 * limit_us microseconds (1..100000) instead of the kernels' one second. The wait runs out, the kernel sets the status
 * word and returns normally (no copy, no tensor memory, nothing in flight). Afterwards attn_b200_device_status(0)
 * returns 1 with tag 99 in attn_b200_last_error(), and every launching entry point refuses with ATTN_B200_ERR_DEVICE
 * until the status is cleared. whole_warp != 0 exercises the converged-warp form of the wait, 0 the single-thread
 * form. No counterpart in the reference (its kernels have no bounded waits).
 */
int attn_b200_selftest_wait(int limit_us, int whole_warp, void* stream);

/* ------------------------------------------------------------------------------------------------------------------
 * Second half: symbols of the per-configuration libraries (one tile configuration of one operation each, built by
 * attention_autotuner_b200.autotuner.Runtime.compile from csrc/kernels/<operation>/profile_code.py). Every such library
 * exports the same six names; the argument lists depend on the operation, so they are given as function-pointer
 * types for dlsym / ctypes users. The two legacy symbols have exactly the reference's argument orders (fp16, the
 * reference's constants, default stream; note Seq_k before Seq_q in kernel_entry and Seq_q before Seq_k in profile);
 * the _ex forms add what the reference hard-codes. dtype and head dimensions are fixed per library.
 *     kernel_entry, kernel_entry_ex : return ATTN_B200_OK or an ATTN_B200_ERR_* code
 *     profile, profile_ex           : return ms per launch, -1 on error
 *     const char* last_error(void); int device_status(int clear);    as attn_b200_last_error / attn_b200_device_status
 * ------------------------------------------------------------------------------------------------------------------ */

/* operation "attn" (reference: csrc/kernels/attention/regfuse/profile_code.py:30 profile, :68 kernel_entry) */
typedef int (*attn_b200_attn_kernel_entry_t)(void* q, void* k, void* v, void* o, int B, int H, int Seq_k, int Seq_q);
typedef float (*attn_b200_attn_profile_t)(void* q, void* k, void* v, void* o, int B, int H, int Seq_q, int Seq_k);
typedef int (*attn_b200_attn_kernel_entry_ex_t)(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                                                int H, int Seq_k, int Seq_q, float scale, int causal, void* stream);
typedef float (*attn_b200_attn_profile_ex_t)(const void* q, const void* k, const void* v, void* o, float* lse, int B, int H,
                                             int Seq_q, int Seq_k, float scale, int causal, void* stream);

/* operation "ret" (reference: csrc/kernels/retnet/regfuse/profile_code.py:30 profile, :72 kernel_entry) */
typedef int (*attn_b200_ret_kernel_entry_t)(void* q, void* k, void* v, void* mask, void* o, float* r, int B, int H, int Seq_k,
                                            int Seq_q);
typedef float (*attn_b200_ret_profile_t)(void* q, void* k, void* v, void* mask, void* o, float* r, int B, int H, int Seq_q,
                                         int Seq_k);
typedef int (*attn_b200_ret_kernel_entry_ex_t)(const void* q, const void* k, const void* v, const void* mask, void* o,
                                               float* r, int B, int H, int Seq_k, int Seq_q, float scale,
                                               const float* decay, int causal, void* stream);
typedef float (*attn_b200_ret_profile_ex_t)(const void* q, const void* k, const void* v, const void* mask, void* o, float* r,
                                            int B, int H, int Seq_q, int Seq_k, float scale, const float* decay, int causal,
                                            void* stream);

/* operation "ret_bwd" (reference: csrc/kernels/retnet/bwd/profile_code.py:50 profile, :98 kernel_entry); dqaccum is
 * scratch of the reference's shape or NULL (see attn_b200_ret_bwd); the _ex forms take its size in bytes last */
typedef int (*attn_b200_ret_bwd_kernel_entry_t)(void* q, void* k, void* v, void* mask, void* dout, float* r, void* dq,
                                                void* dk, void* dv, float* dqaccum, int B, int H, int Seq_k, int Seq_q);
typedef float (*attn_b200_ret_bwd_profile_t)(void* q, void* k, void* v, void* mask, void* dout, float* r, void* dq, void* dk,
                                             void* dv, float* dqaccum, int B, int H, int Seq_q, int Seq_k);
typedef int (*attn_b200_ret_bwd_kernel_entry_ex_t)(const void* q, const void* k, const void* v, const void* mask,
                                                   const void* dout, const float* r, void* dq, void* dk, void* dv,
                                                   float* dqaccum, int B, int H, int Seq_k, int Seq_q, float scale,
                                                   const float* decay, int causal, void* stream, size_t dqaccum_bytes);
typedef float (*attn_b200_ret_bwd_profile_ex_t)(const void* q, const void* k, const void* v, const void* mask,
                                                const void* dout, const float* r, void* dq, void* dk, void* dv,
                                                float* dqaccum, int B, int H, int Seq_q, int Seq_k, float scale,
                                                const float* decay, int causal, void* stream, size_t dqaccum_bytes);

#ifdef __cplusplus
}
#endif

#endif /* ATTN_B200_H_ */
