// Stand-alone comparison harness: cuBLAS (kernel 0) against libneogemm through its C ABI
// (kernel 1) on the same device buffers.  It plays the role of the reference's cublass/matmul.cu
// (kernel table matmul.cu:45-51, seeded operands :31,53-59, verification :61-75, event timing
// :170-183), with these differences: any M, N, K from the command line (the reference's lda/ldc
// are only right for square sizes, matmul.cu:36-37), operands N(0,1)/sqrt(K), verification that
// actually runs for every kernel (the reference's is guarded off, matmul.cu:144), a check against
// a CPU fp32 product on sampled elements, and the per-CTA phase timers filled in
// (the reference only reserves the buffer, matmul.cu:99-106).
//
//   ./matmul [M N K] [--iters 200] [--timers]
#include <cublas_v2.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "../include/neogemm.h"

#define CUDA_OK(call)                                                                      \
  do {                                                                                     \
    cudaError_t e_ = (call);                                                               \
    if (e_ != cudaSuccess) {                                                               \
      std::fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__,   \
                   __LINE__);                                                              \
      std::exit(1);                                                                        \
    }                                                                                      \
  } while (0)

static cublasHandle_t g_handle;

// Row-major C[M,N] = A[M,K] * B[N,K]^T.  In cuBLAS's column-major view that is
// C^T[N,M] = B'[N,K]... : op(B)=T on the K x N column-major view of B, op(A)=N on the K x M view of A.
static void run_cublas(int M, int N, int K, const __nv_bfloat16* A, const __nv_bfloat16* B,
                       __nv_bfloat16* C) {
  const float alpha = 1.0f, beta = 0.0f;
  cublasStatus_t st = cublasGemmEx(g_handle, CUBLAS_OP_T, CUBLAS_OP_N, N, M, K, &alpha, B,
                                   CUDA_R_16BF, K, A, CUDA_R_16BF, K, &beta, C, CUDA_R_16BF, N,
                                   CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
  if (st != CUBLAS_STATUS_SUCCESS) {
    std::fprintf(stderr, "cublasGemmEx failed: %d\n", static_cast<int>(st));
    std::exit(1);
  }
}

static void run_neogemm(int M, int N, int K, const __nv_bfloat16* A, const __nv_bfloat16* B,
                        __nv_bfloat16* C) {
  const int rc = neogemm_bf16_nt(A, B, C, M, N, K, K, K, N, 0, nullptr, 0, nullptr);
  if (rc != NEOGEMM_OK) {
    std::fprintf(stderr, "neogemm_bf16_nt: %s\n", neogemm_status_str(rc));
    std::exit(1);
  }
}

static void run_kernel(int id, int M, int N, int K, const __nv_bfloat16* A,
                       const __nv_bfloat16* B, __nv_bfloat16* C) {
  if (id == 0) run_cublas(M, N, K, A, B, C);
  else run_neogemm(M, N, K, A, B, C);
}

static void randomize(std::vector<__nv_bfloat16>& v, unsigned seed, float scale) {
  std::mt19937 gen(seed);
  std::normal_distribution<float> dist(0.0f, 1.0f);
  for (auto& x : v) x = __float2bfloat16(dist(gen) * scale);
}

int main(int argc, char** argv) {
  int M = 4096, N = 4096, K = 4096, iters = 200;
  bool timers = false;
  int pos = 0;
  for (int i = 1; i < argc; ++i) {
    if (!std::strcmp(argv[i], "--iters") && i + 1 < argc) iters = std::atoi(argv[++i]);
    else if (!std::strcmp(argv[i], "--timers")) timers = true;
    else if (pos == 0) { M = std::atoi(argv[i]); ++pos; }
    else if (pos == 1) { N = std::atoi(argv[i]); ++pos; }
    else if (pos == 2) { K = std::atoi(argv[i]); ++pos; }
  }
  std::printf("M=%d N=%d K=%d iters=%d\n", M, N, K, iters);
  if (cublasCreate(&g_handle) != CUBLAS_STATUS_SUCCESS) {
    std::fprintf(stderr, "cublasCreate failed\n");
    return 1;
  }
  std::vector<__nv_bfloat16> hA(static_cast<size_t>(M) * K), hB(static_cast<size_t>(N) * K);
  std::vector<__nv_bfloat16> hC0(static_cast<size_t>(M) * N), hC1(static_cast<size_t>(M) * N);
  const float scale = 1.0f / std::sqrt(static_cast<float>(K));
  randomize(hA, 69, scale);
  randomize(hB, 70, scale);
  __nv_bfloat16 *dA, *dB, *dC0, *dC1;
  CUDA_OK(cudaMalloc(&dA, hA.size() * 2));
  CUDA_OK(cudaMalloc(&dB, hB.size() * 2));
  CUDA_OK(cudaMalloc(&dC0, hC0.size() * 2));
  CUDA_OK(cudaMalloc(&dC1, hC1.size() * 2));
  CUDA_OK(cudaMemcpy(dA, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice));
  CUDA_OK(cudaMemcpy(dB, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice));
  CUDA_OK(cudaMemset(dC0, 0xff, hC0.size() * 2));   // NaN poison
  CUDA_OK(cudaMemset(dC1, 0xff, hC1.size() * 2));

  // ---- verification: ours against cuBLAS everywhere, both against a CPU fp32 product on samples
  run_kernel(0, M, N, K, dA, dB, dC0);
  run_kernel(1, M, N, K, dA, dB, dC1);
  CUDA_OK(cudaDeviceSynchronize());
  int dev_status[4] = {0, 0, 0, 0};
  neogemm_device_status(dev_status);
  if (dev_status[0] != 0) {
    std::fprintf(stderr, "device-side error %d (CTA %d, segment %d, aux %d)\n", dev_status[0],
                 dev_status[1], dev_status[2], dev_status[3]);
    return 1;
  }
  CUDA_OK(cudaMemcpy(hC0.data(), dC0, hC0.size() * 2, cudaMemcpyDeviceToHost));
  CUDA_OK(cudaMemcpy(hC1.data(), dC1, hC1.size() * 2, cudaMemcpyDeviceToHost));
  double max_diff = 0.0;
  size_t differing = 0, bad = 0;
  for (size_t i = 0; i < hC0.size(); ++i) {
    const float a = __bfloat162float(hC0[i]), b = __bfloat162float(hC1[i]);
    if (!(std::isfinite(a) && std::isfinite(b))) { ++bad; continue; }
    const double d = std::fabs(static_cast<double>(a) - b);
    if (d > 0) ++differing;
    if (d > max_diff) max_diff = d;
    if (d > 1e-2 + 1e-2 * std::fabs(a)) ++bad;
  }
  std::printf("ours vs cuBLAS: max |diff| %.3e, %zu of %zu elements differ (last-bit rounding), "
              "%zu outside rtol=atol=1e-2\n", max_diff, differing, hC0.size(), bad);
  std::mt19937 pick(7);
  double max_cpu = 0.0;
  for (int s = 0; s < 2048; ++s) {
    const size_t i = pick() % static_cast<size_t>(M), j = pick() % static_cast<size_t>(N);
    float acc = 0.0f;
    for (int k = 0; k < K; ++k)
      acc += __bfloat162float(hA[i * K + k]) * __bfloat162float(hB[j * K + k]);
    const double d = std::fabs(static_cast<double>(acc) - __bfloat162float(hC1[i * N + j]));
    if (d > max_cpu) max_cpu = d;
    if (d > 1e-2 + 1e-2 * std::fabs(acc)) ++bad;
  }
  std::printf("ours vs CPU fp32 on 2048 samples: max |diff| %.3e\n", max_cpu);
  if (bad != 0) {
    std::printf("Divergence! %zu elements out of tolerance\n", bad);
    return 1;
  }

  // ---- timing, interleaved so that both see the same thermal state
  cudaEvent_t e0, e1;
  CUDA_OK(cudaEventCreate(&e0));
  CUDA_OK(cudaEventCreate(&e1));
  const double flops = 2.0 * M * N * K;
  for (int round = 0; round < 3; ++round) {
    for (int id = 0; id < 2; ++id) {
      __nv_bfloat16* out = id == 0 ? dC0 : dC1;
      for (int w = 0; w < 5; ++w) run_kernel(id, M, N, K, dA, dB, out);
      CUDA_OK(cudaEventRecord(e0));
      for (int it = 0; it < iters; ++it) run_kernel(id, M, N, K, dA, dB, out);
      CUDA_OK(cudaEventRecord(e1));
      CUDA_OK(cudaEventSynchronize(e1));
      float ms = 0.0f;
      CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
      const double s = ms / 1e3 / iters;
      std::printf("round %d  %-8s %.6f s/iter  %.1f TFLOPS\n", round, id == 0 ? "cuBLAS" : "neogemm",
                  s, flops / s / 1e12);
    }
  }

  // ---- per-CTA phase timers of one launch (filled-in version of the reference's DB records)
  if (timers) {
    int cfg[8];
    neogemm_last_config(cfg);
    const int ctas = cfg[5];
    long long* dT;
    CUDA_OK(cudaMalloc(&dT, static_cast<size_t>(ctas) * 16 * sizeof(long long)));
    CUDA_OK(cudaMemset(dT, 0, static_cast<size_t>(ctas) * 16 * sizeof(long long)));
    neogemm_set_phase_timers(dT, static_cast<size_t>(ctas) * 16 * sizeof(long long));
    run_kernel(1, M, N, K, dA, dB, dC1);
    CUDA_OK(cudaDeviceSynchronize());
    neogemm_set_phase_timers(nullptr, 0);
    std::vector<long long> t(static_cast<size_t>(ctas) * 16);
    CUDA_OK(cudaMemcpy(t.data(), dT, t.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    double load_wait = 0, load_loop = 0, mma_wait = 0, mma_loop = 0, epi_wait = 0, epi_loop = 0;
    int leaders = 0;
    for (int c = 0; c < ctas; ++c) {
      const long long* r = &t[static_cast<size_t>(c) * 16];
      load_wait += r[0]; load_loop += r[1]; epi_wait += r[5]; epi_loop += r[6];
      if (r[4] > 0) { mma_wait += r[2] + r[3]; mma_loop += r[4]; ++leaders; }
    }
    std::printf("phase timers over %d CTAs (%d issue MMAs), config: %d CTA/tile, N=%d, %d stages\n",
                ctas, leaders, cfg[0], cfg[1], cfg[2]);
    std::printf("  load   : loop %.0f cycles/CTA, waiting for a free slot %.1f %%\n",
                load_loop / ctas, 100.0 * load_wait / load_loop);
    std::printf("  compute: loop %.0f cycles/CTA, waiting for operands or TMEM %.1f %%\n",
                mma_loop / leaders, 100.0 * mma_wait / mma_loop);
    std::printf("  store  : loop %.0f cycles/CTA, waiting for an accumulator %.1f %%\n",
                epi_loop / ctas, 100.0 * epi_wait / epi_loop);
    cudaFree(dT);
  }
  cudaFree(dA); cudaFree(dB); cudaFree(dC0); cudaFree(dC1);
  cublasDestroy(g_handle);
  return 0;
}
