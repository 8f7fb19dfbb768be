/* CPU oracle for the BF16 GEMM path.  TEST INFRASTRUCTURE ONLY: tests, the smoke check and the
 * CPU-baseline leg of the benchmark may call this; the library never does.
 *
 * PARITY UNPINNED by the reference: it ships no golden vectors, known-answer tests or fixtures
 * for this path (only printed comparisons, benchmark.py:33-53), its Hopper kernels cannot run on
 * sm_100 and its Blackwell files do not compile, so nothing of the reference can be executed to
 * pin this restatement.  It is pinned instead against itself three ways (this scalar loop, an
 * fp64-accumulating loop, and torch's fp32 CPU matmul) in tests/test_oracle.py.
 *
 * What it restates:
 *   - operands are bf16, products accumulate in fp32 over the whole K range with no alpha/beta
 *     (wgmma m64n64k16 f32.bf16.bf16 with ScaleD = 1 over every k-tile, neogemmV02.cu:159,222-225);
 *   - the result is rounded to bf16 with round-to-nearest-even (__float2bfloat16,
 *     neogemmV02.cu:244);
 *   - M, K come from A and N from B's row count (nemgemmV03.cu:344-346), C = A * B^T
 *     (benchmark.py:18);
 *   - the reference stores C column-major, element (i,j) at C[j*M + i] (neogemmV02.cu:236,242),
 *     which benchmark.py:25 undoes with a transposed view; row-major output is offered as well.
 * The order of the fp32 additions inside the tensor core is not specified by the hardware, so
 * device results may differ from this loop in the last bf16 bit on a small fraction of elements;
 * the tests state that tolerance.
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round-to-nearest-even, NaN kept quiet: the rounding of __float2bfloat16_rn. */
static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x0040u);
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return (uint16_t)(u >> 16);
}

/* C = A * B^T, fp32 accumulation in k order.  A [M,K] pitch lda, B [N,K] pitch ldb (elements).
 * c_col_major != 0: C(i,j) at C[j*ldc + i]; else at C[i*ldc + j].
 * Rows [row_begin, row_end) of A only, so that callers can split the work over threads. */
void oracle_gemm_bf16_nt(const uint16_t* A, const uint16_t* B, uint16_t* C, int64_t M, int64_t N,
                         int64_t K, int64_t lda, int64_t ldb, int64_t ldc, int c_col_major,
                         int64_t row_begin, int64_t row_end) {
  (void)M;
  for (int64_t i = row_begin; i < row_end; ++i) {
    for (int64_t j = 0; j < N; ++j) {
      float acc = 0.0f;
      const uint16_t* a = A + i * lda;
      const uint16_t* b = B + j * ldb;
      for (int64_t k = 0; k < K; ++k) acc += bf16_to_f32(a[k]) * bf16_to_f32(b[k]);
      if (c_col_major) C[j * ldc + i] = f32_to_bf16_rne(acc);
      else C[i * ldc + j] = f32_to_bf16_rne(acc);
    }
  }
}

/* Same product accumulated in fp64 and returned unrounded (row-major fp64 [M,N]): the yardstick
 * the fp32 restatements are themselves checked against. */
void oracle_gemm_f64(const uint16_t* A, const uint16_t* B, double* C, int64_t M, int64_t N,
                     int64_t K, int64_t lda, int64_t ldb) {
  for (int64_t i = 0; i < M; ++i) {
    for (int64_t j = 0; j < N; ++j) {
      double acc = 0.0;
      for (int64_t k = 0; k < K; ++k)
        acc += (double)bf16_to_f32(A[i * lda + k]) * (double)bf16_to_f32(B[j * ldb + k]);
      C[i * N + j] = acc;
    }
  }
}

/* Exposed so the tests can check the rounding rule on its own. */
uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }
float oracle_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }
