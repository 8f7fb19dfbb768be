"""GPU: the entry point that never allocates (neogemm_bf16_nt_noalloc) against the regular one.

Some callers cannot let a library allocate when they multiply: their own pool already owns the
device's memory, or they run where an allocation's latency (or its failure) is not acceptable.
For them the library carries a fixed 32 MiB scratch array, and this entry point uses it instead of
a cudaMalloc'ed stream-K workspace.  The test calls it through the C ABI twice in a row on a
skinny (stream-K) shape and on a large (data-parallel) one and compares with neogemm_bf16_nt on
the same operands, with the gates every other parity test uses (at most one bf16 ulp apart, at
least 98 % of elements bit-equal; in practice the bits are identical because both paths sum in
the same fixed order).  It also checks that a shape beyond the fixed scratch is refused.

Collected last on purpose: a run that stops at the first failure has then run everything else.
"""
import pytest
import torch

from gemm_b200 import ops
from gemm_b200._lib import lib
from gemm_b200.inputs import make_problem
from oracle import oracle

pytestmark = pytest.mark.gpu


def _noalloc(A, B, C, M, N, K, col_major=False):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.neogemm_bf16_nt_noalloc(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, K, K,
                                       M if col_major else N, 1 if col_major else 0, stream)


@pytest.mark.parametrize("shape", [(64, 3584, 2048), (16, 28672, 8192), (128, 28672, 8192),
                                   (1024, 768, 512)])
def test_noalloc_matches_regular_entry_point_twice(shape):
    M, N, K = shape
    A, B = make_problem(M, N, K, seed=4242)
    dA, dB = A.cuda(), B.cuda()
    want = ops.matmul(dA, dB)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    ref = oracle.gemm_fp32(A, B)
    for call in range(2):
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert _noalloc(dA, dB, got, M, N, K) == 0
        torch.cuda.synchronize()
        s = oracle.compare(got, want.float().cpu())
        assert s["finite"] and s["max_ulp"] <= 1 and s["near_zero_ok"] and \
            s["bit_equal_frac"] >= 0.98, (call, shape, s)
        oracle.assert_parity(got, ref, f"noalloc call {call} {shape}")


def test_noalloc_column_major_like_the_reference():
    M, N, K = 48, 2048, 1024
    A, B = make_problem(M, N, K, seed=77)
    dA, dB = A.cuda(), B.cuda()
    for _ in range(2):
        C = torch.full((N, M), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert _noalloc(dA, dB, C, M, N, K, col_major=True) == 0
        torch.cuda.synchronize()
        oracle.assert_parity(C.t(), oracle.gemm_fp32(A, B), "noalloc column-major")


def test_noalloc_refuses_shapes_beyond_its_fixed_scratch():
    # 448 tiles of 128 x 128 fp32 partials, two contributors each: 58.7 MB > 32 MiB.  The refusal
    # comes from planning, before any operand is touched, so small dummy buffers are enough.
    dummy = torch.zeros(1 << 16, dtype=torch.bfloat16, device="cuda")
    rc = lib.neogemm_bf16_nt_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                     128, 2 * 28672, 8192, 8192, 8192, 2 * 28672, 0, None)
    assert rc == 6, f"expected NEOGEMM_ERR_WORKSPACE, got {rc}"
    # and the usual argument checks still apply
    assert lib.neogemm_bf16_nt_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                       8, 8, 12, 16, 16, 8, 0, None) == 2
