// Standalone C++ micro-benchmark of the RetNet parallel forward and backward chain kernels (single-CTA and CTA-pair
// flavours), instantiated here from the kernel headers. Same role as the reference's benchmarks/retnet/retnet.cu
// and retnet_bwd.cu (test_regfuse_retnet / test_smemfuse_retnet / the backward test on ProblemShape records).
//
//   retnet_bench [--B 4 --H 8 --Seq_q 2048 --Seq_k 2048] [--mask] [--bwd]
//
// Head dimensions 256 / 512 (the benchmark configuration). Default: per-head decay built in registers; --mask hands
// the same decay mask over as the reference's [H, Seq_q, Seq_k] 16-bit tensor. --bwd times forward + backward.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../csrc/chain_launch.cuh"
#include "bench_common.cuh"

using namespace ab200;

constexpr int kDqk = 256, kDv = 512;

template <bool PAIR>
static BenchResult time_flavour(const RetArgs& a, bool bwd) {
  return do_bench([&]() -> int {
    int rc = ret_fwd_launch<kDqk, 256, false, PAIR>(a, nullptr);
    if (rc == 0 && bwd) rc = ret_bwd_launch<kDqk, kDv, 256, 256, false, PAIR>(a, nullptr);
    if (rc != 0) fprintf(stderr, "launch failed: %s\n", error_buffer());
    return rc;
  });
}

int main(int argc, char** argv) {
  Args args{argc, argv};
  ProblemShape s(args.num("--B", 4), args.num("--H", 8), args.num("--Seq_q", 2048), args.num("--Seq_k", 2048));
  const bool use_mask = args.flag("--mask"), bwd = args.flag("--bwd");
  const size_t bh = static_cast<size_t>(s.B) * s.H;
  const size_t nq = bh * s.Seq_q * kDqk, nk = bh * s.Seq_k * kDqk, nv = bh * s.Seq_k * kDv, no = bh * s.Seq_q * kDv;
  void *q, *k, *v, *o, *dout, *dq, *dk, *dvo, *mask = nullptr;
  float *r, *decay;
  BENCH_CUDA(cudaMalloc(&q, nq * 2));
  BENCH_CUDA(cudaMalloc(&k, nk * 2));
  BENCH_CUDA(cudaMalloc(&v, nv * 2));
  BENCH_CUDA(cudaMalloc(&o, no * 2));
  BENCH_CUDA(cudaMalloc(&dout, no * 2));
  BENCH_CUDA(cudaMalloc(&dq, nq * 2));
  BENCH_CUDA(cudaMalloc(&dk, nk * 2));
  BENCH_CUDA(cudaMalloc(&dvo, nv * 2));
  BENCH_CUDA(cudaMalloc(&r, bh * s.Seq_q * sizeof(float)));
  BENCH_CUDA(cudaMalloc(&decay, s.H * sizeof(float)));
  fill_normal(q, nq, 1, false);
  fill_normal(k, nk, 2, false);
  fill_normal(v, nv, 3, false);
  fill_normal(dout, no, 4, false);
  std::vector<float> gam(s.H);
  for (int h = 0; h < s.H; ++h) gam[h] = 1.0f - exp2f(-5.0f - h);
  BENCH_CUDA(cudaMemcpy(decay, gam.data(), s.H * sizeof(float), cudaMemcpyHostToDevice));
  if (use_mask) {
    BENCH_CUDA(cudaMalloc(&mask, static_cast<size_t>(s.H) * s.Seq_q * s.Seq_k * 2));
    bench_fill_decay_mask<false><<<148 * 8, 256>>>(static_cast<uint16_t*>(mask), s.H, s.Seq_q, s.Seq_k);
    BENCH_CUDA(cudaGetLastError());
  }
  RetArgs a{};
  a.q = q; a.k = k; a.v = v; a.mask = mask; a.decay = use_mask ? nullptr : decay; a.o = o; a.r = r;
  a.dout = dout; a.dq = dq; a.dk = dk; a.dv_out = dvo;
  a.BH = s.B * s.H; a.H = s.H; a.Lq = s.Seq_q; a.Lkv = s.Seq_k; a.dqk = kDqk; a.dv = kDv;
  a.scale = 1.0f / sqrtf(static_cast<float>(kDqk));
  a.causal = 1;
  const double pairs = attention_pairs(s.Seq_q, s.Seq_k, true);
  const double flops = 2.0 * s.B * s.H * pairs * ((kDqk + kDv) + (bwd ? (3 * kDqk + 2 * kDv) : 0));
  const char* what = bwd ? (use_mask ? "retnet fwd+bwd (mask tensor)" : "retnet fwd+bwd (decay)")
                         : (use_mask ? "retnet fwd (mask tensor)" : "retnet fwd (decay)");
  print_result(what, "cta_pair dv_chunk=256 dq_chunk=256", s, kDqk, kDv, time_flavour<true>(a, bwd), flops);
  print_result(what, "single CTA dv_chunk=256 dq_chunk=256", s, kDqk, kDv, time_flavour<false>(a, bwd), flops);
  int det = 0;
  if (read_device_status(1, &det) != 0) {
    fprintf(stderr, "device status: %s\n", error_buffer());
    return 3;
  }
  return 0;
}
