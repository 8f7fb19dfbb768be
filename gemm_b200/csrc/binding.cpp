// PyTorch binding: module `neoGEMM`, function `neoGemmV1(A, B, C)` - the reference's operator
// surface (nemgemmV03.cu:343-398; legacy `neogemm`, neogemmV02.cu:262-306) - on top of the C ABI
// of libneogemm.so.  Only this file sees torch headers; it is compiled by the host compiler.
//
// Differences from the reference binding, all on the safe side:
//   * dtype, device, rank, contiguity and shape agreement are checked (the reference reads raw
//     data_ptr<at::BFloat16>() unchecked, nemgemmV03.cu:349-351);
//   * the launch goes to torch's current stream on A's device (the reference uses the legacy
//     default stream of whatever device is current, nemgemmV03.cu:383);
//   * failures raise RuntimeError (the reference prints to stderr, nemgemmV03.cu:387-390).
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include "neogemm.h"

namespace {

void check_matrix(const torch::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (there is no CPU path)");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
  TORCH_CHECK(t.dim() == 2, name, " must be 2-D");
  TORCH_CHECK(t.size(1) <= 1 || t.stride(1) == 1, name, " must have contiguous rows");
}

int64_t row_pitch(const torch::Tensor& t) {
  return t.size(0) > 1 ? t.stride(0) : std::max<int64_t>(t.size(1), 1);
}

void run(const torch::Tensor& A, const torch::Tensor& B, void* C, int64_t ldc, bool col_major) {
  const int64_t M = A.size(0), K = A.size(1), N = B.size(0);
  c10::cuda::CUDAGuard guard(A.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(A.device().index()).stream();
  const int rc = neogemm_bf16_nt(A.data_ptr(), B.data_ptr(), C, M, N, K, row_pitch(A),
                                 row_pitch(B), ldc, col_major ? 1 : 0, nullptr, 0,
                                 static_cast<void*>(stream));
  TORCH_CHECK(rc == NEOGEMM_OK, "neoGEMM: ", neogemm_status_str(rc));
}

void check_pair(const torch::Tensor& A, const torch::Tensor& B) {
  check_matrix(A, "A");
  check_matrix(B, "B");
  TORCH_CHECK(A.device() == B.device(), "A and B must be on the same device");
  TORCH_CHECK(A.size(1) == B.size(1), "A is [M,K] and B is [N,K]: their K differ");
}

// C <- A * B^T stored column-major in C (element (i,j) at j*M + i), as the reference does.
void neoGemmV1(torch::Tensor A, torch::Tensor B, torch::Tensor C) {
  check_pair(A, B);
  TORCH_CHECK(C.is_cuda() && C.scalar_type() == at::kBFloat16, "C must be a CUDA bfloat16 tensor");
  TORCH_CHECK(C.device() == A.device(), "C must be on the same device as A and B");
  TORCH_CHECK(C.is_contiguous() && C.numel() == A.size(0) * B.size(0),
              "C must be contiguous with M*N elements");
  run(A, B, C.data_ptr(), std::max<int64_t>(A.size(0), 1), true);
}

// Row-major convenience: returns C[M,N].
torch::Tensor matmul(torch::Tensor A, torch::Tensor B) {
  check_pair(A, B);
  auto C = torch::empty({A.size(0), B.size(0)}, A.options());
  run(A, B, C.data_ptr(), std::max<int64_t>(B.size(0), 1), false);
  return C;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "BF16 GEMM C = A * B^T for B200 (sm_100a): TMA + tcgen05 + TMEM";
  m.def("neoGemmV1", &neoGemmV1, "C <- A * B^T, column-major in C (reference-compatible)",
        pybind11::arg("A"), pybind11::arg("B"), pybind11::arg("C"));
  m.def("neogemm", &neoGemmV1, "legacy name of neoGemmV1", pybind11::arg("A"),
        pybind11::arg("B"), pybind11::arg("C"));
  m.def("matmul", &matmul, "returns row-major C[M,N] = A * B^T", pybind11::arg("A"),
        pybind11::arg("B"));
}
