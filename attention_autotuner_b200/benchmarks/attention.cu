// Standalone C++ micro-benchmark of the flash-attention forward kernels: times named tile configurations of
// fa_fwd_sm100_kernel / fa_fwd_pair_sm100_kernel, instantiated here from the kernel headers, on one problem shape.
// Same role as the reference's benchmarks/attention.cu:34-304 (test_regfuse_attention / test_smemfuse_attention
// instantiated with ImplementShape* records and timed on ProblemShape(4, 8, 2048, 2048)).
//
//   attention_bench [--B 4 --H 8 --Seq_q 2048 --Seq_k 2048] [--d 128] [--causal] [--bf16] [--check]
//
// --check compares row 0 of slice 0 of the first configuration's output with a plain fp32 evaluation on the host.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../csrc/fa_fwd_launch.cuh"
#include "bench_common.cuh"

using namespace ab200;

template <class Cfg, bool PAIR = false>
static BenchResult time_config(const ProblemShape& s, const void* q, const void* k, const void* v, void* o, float scale, int causal) {
  FaFwdArgs a{q, k, v, o, nullptr, s.B * s.H, s.Seq_q, s.Seq_k, Cfg::DV, scale, causal};
  return do_bench([&]() -> int {
    int rc;
    if constexpr (PAIR) rc = fa_fwd_pair_launch<Cfg>(a, nullptr);
    else rc = fa_fwd_launch<Cfg>(a, nullptr);
    if (rc != 0) fprintf(stderr, "launch failed: %s\n", error_buffer());
    return rc;
  });
}

static float to_float(uint16_t bits, bool bf16) {
  if (bf16) {
    uint32_t u = static_cast<uint32_t>(bits) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
  }
  __half h;
  memcpy(&h, &bits, 2);
  return __half2float(h);
}

// row 0 of (batch 0, head 0) on the host in fp32: max abs difference to the kernel's output
static double check_row0(const ProblemShape& s, int d, bool bf16, const void* q, const void* k, const void* v, const void* o, float scale) {
  std::vector<uint16_t> hq(d), hk(static_cast<size_t>(s.Seq_k) * d), hv(static_cast<size_t>(s.Seq_k) * d), ho(d);
  BENCH_CUDA(cudaMemcpy(hq.data(), q, d * 2, cudaMemcpyDeviceToHost));
  BENCH_CUDA(cudaMemcpy(hk.data(), k, hk.size() * 2, cudaMemcpyDeviceToHost));
  BENCH_CUDA(cudaMemcpy(hv.data(), v, hv.size() * 2, cudaMemcpyDeviceToHost));
  BENCH_CUDA(cudaMemcpy(ho.data(), o, d * 2, cudaMemcpyDeviceToHost));
  const int visible = s.Seq_k;  // non-causal check (row 0 under a causal mask sees Seq_k - Seq_q + 1 keys)
  std::vector<double> p(visible);
  double mx = -1e300;
  for (int j = 0; j < visible; ++j) {
    double acc = 0.0;
    for (int c = 0; c < d; ++c) acc += static_cast<double>(to_float(hq[c], bf16)) * to_float(hk[static_cast<size_t>(j) * d + c], bf16);
    p[j] = acc * scale;
    mx = std::max(mx, p[j]);
  }
  double l = 0.0;
  for (int j = 0; j < visible; ++j) { p[j] = exp(p[j] - mx); l += p[j]; }
  double worst = 0.0;
  for (int c = 0; c < d; ++c) {
    double acc = 0.0;
    for (int j = 0; j < visible; ++j) acc += p[j] * to_float(hv[static_cast<size_t>(j) * d + c], bf16);
    worst = std::max(worst, fabs(acc / l - to_float(ho[c], bf16)));
  }
  return worst;
}

template <bool BF16>
static int run(const Args& args) {
  ProblemShape s(args.num("--B", 4), args.num("--H", 8), args.num("--Seq_q", 2048), args.num("--Seq_k", 2048));
  const int d = args.num("--d", 128);
  const int causal = args.flag("--causal") ? 1 : 0;
  const float scale = 1.0f / sqrtf(static_cast<float>(d));
  const size_t nq = static_cast<size_t>(s.B) * s.H * s.Seq_q * d, nk = static_cast<size_t>(s.B) * s.H * s.Seq_k * d;
  void *q, *k, *v, *o;
  BENCH_CUDA(cudaMalloc(&q, nq * 2));
  BENCH_CUDA(cudaMalloc(&k, nk * 2));
  BENCH_CUDA(cudaMalloc(&v, nk * 2));
  BENCH_CUDA(cudaMalloc(&o, nq * 2));
  fill_normal(q, nq, 1, BF16);
  fill_normal(k, nk, 2, BF16);
  fill_normal(v, nk, 3, BF16);
  const double flops = 2.0 * s.B * s.H * attention_pairs(s.Seq_q, s.Seq_k, causal) * (d + d);
  const char* what = causal ? "attention fwd causal" : "attention fwd";
  if (d == 128) {
    // two ping-ponging query tiles with K/V rings of 3, 4 and 5 tiles; one query tile; a CTA pair
    BenchResult r = time_config<FaFwdConfig<128, 128, 2, 4, BF16>>(s, q, k, v, o, scale, causal);
    print_result(what, "q_tiles=2 kv_stages=4", s, d, d, r, flops);
    if (args.flag("--check") && !causal) {
      const double err = check_row0(s, d, BF16, q, k, v, o, scale);
      printf("check: max abs error of row 0 against the host evaluation %.3e (%s)\n", err, err < (BF16 ? 1.6e-2 : 2e-3) ? "ok" : "FAIL");
      if (!(err < (BF16 ? 1.6e-2 : 2e-3))) return 1;
    }
    print_result(what, "q_tiles=2 kv_stages=3", s, d, d, time_config<FaFwdConfig<128, 128, 2, 3, BF16>>(s, q, k, v, o, scale, causal), flops);
    print_result(what, "q_tiles=2 kv_stages=5", s, d, d, time_config<FaFwdConfig<128, 128, 2, 5, BF16>>(s, q, k, v, o, scale, causal), flops);
    print_result(what, "q_tiles=1 kv_stages=4", s, d, d, time_config<FaFwdConfig<128, 128, 1, 4, BF16>>(s, q, k, v, o, scale, causal), flops);
    print_result(what, "cta_pair kv_stages=4", s, d, d, time_config<FaPairConfig<128, 8, BF16>, true>(s, q, k, v, o, scale, causal), flops);
  } else if (d == 64) {
    BenchResult r = time_config<FaFwdConfig<64, 64, 2, 4, BF16>>(s, q, k, v, o, scale, causal);
    print_result(what, "q_tiles=2 kv_stages=4", s, d, d, r, flops);
    if (args.flag("--check") && !causal) {
      const double err = check_row0(s, d, BF16, q, k, v, o, scale);
      printf("check: max abs error of row 0 against the host evaluation %.3e (%s)\n", err, err < (BF16 ? 1.6e-2 : 2e-3) ? "ok" : "FAIL");
      if (!(err < (BF16 ? 1.6e-2 : 2e-3))) return 1;
    }
    print_result(what, "q_tiles=2 kv_stages=6", s, d, d, time_config<FaFwdConfig<64, 64, 2, 6, BF16>>(s, q, k, v, o, scale, causal), flops);
  } else {
    fprintf(stderr, "--d must be 64 or 128\n");
    return 2;
  }
  int det = 0;
  if (read_device_status(1, &det) != 0) {
    fprintf(stderr, "device status: %s\n", error_buffer());
    return 3;
  }
  cudaFree(q); cudaFree(k); cudaFree(v); cudaFree(o);
  return 0;
}

int main(int argc, char** argv) {
  Args args{argc, argv};
  return args.flag("--bf16") ? run<true>(args) : run<false>(args);
}
