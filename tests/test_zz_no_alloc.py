"""GPU: the entry point that never allocates (neogemm_bf16_nt_noalloc) against the regular one.

Some callers cannot let a library allocate when they multiply: their own pool already owns the
device's memory, or they run where an allocation's latency (or its failure) is not acceptable.
For them the library carries a fixed 32 MiB scratch array, and this entry point uses it instead of
a cudaMalloc'ed stream-K workspace.  The tests call it through the C ABI twice in a row and
compare with neogemm_bf16_nt on the same operands, with the gates every other parity test uses
(at most one bf16 ulp apart, at least 98 % of elements bit-equal; in practice the bits are
identical because both paths sum in the same fixed order).  Shapes that are meant to exercise the
fixed array assert that the plan really cut tiles (stream_k == 1); others cover the plans that
need no scratch.  Also checked: a shape beyond the fixed scratch is refused, and a device-side
error of this entry point is visible, sticky and clearable.

Collected last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

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


def _noalloc_status():
    out = (ctypes.c_int * 4)()
    assert lib.neogemm_noalloc_status(out, torch.cuda.current_stream().cuda_stream) == 0
    return tuple(out)


def _check_twice(shape, uses_scratch, seed=4242):
    M, N, K = shape
    A, B = make_problem(M, N, K, seed=seed)
    dA, dB = A.cuda(), B.cuda()
    want = ops.matmul(dA, dB)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    ref = oracle.gemm_fp32(A, B)
    for call in range(2):
        got = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert _noalloc(dA, dB, got, M, N, K) == 0
        cfg = ops.last_config()
        assert cfg["stream_k"] == (1 if uses_scratch else 0), (shape, cfg)
        torch.cuda.synchronize()
        assert _noalloc_status()[0] == 0
        s = oracle.compare(got, want.float().cpu())
        assert s["finite"] and s["max_ulp"] <= 1 and s["near_zero_ok"] and \
            s["bit_equal_frac"] >= 0.98, (call, shape, s)
        oracle.assert_parity(got, ref, f"noalloc call {call} {shape}")


def test_noalloc_init_is_repeatable():
    assert lib.neogemm_noalloc_init() == 0
    assert lib.neogemm_noalloc_init() == 0
    assert _noalloc_status() == (0, 0, 0, 0)


# Cut tiles with their partial sums in the fixed array: uniform k-chunks (64 x 3584 x 2048: 28
# tiles in 4 chunks; 16 x 3584 x 8192: 28 tiles in 5 chunks) and contiguous ranges with pieces
# claimed at run time (16 x 40960 x 4096: 320 tiles on 148 CTAs, one 16-k-block piece per tile).
@pytest.mark.parametrize("shape", [(64, 3584, 2048), (16, 3584, 8192), (16, 40960, 4096)])
def test_noalloc_with_scratch_matches_regular_entry_point_twice(shape):
    _check_twice(shape, uses_scratch=True)


# Plans that need no scratch: one wave of whole tall tiles (the decode shapes)
# and a data-parallel TMA-store plan.
@pytest.mark.parametrize("shape", [(16, 28672, 8192), (128, 28672, 8192), (1024, 768, 512)])
def test_noalloc_without_scratch_matches_regular_entry_point_twice(shape):
    _check_twice(shape, uses_scratch=False)


def test_noalloc_two_scratch_shapes_back_to_back():
    # The array keeps the previous call's partial sums: a different shape right behind it, on
    # the same stream and without a host synchronisation in between, must not see them.
    shapes = [(64, 3584, 2048), (32, 7168, 4096), (64, 3584, 2048)]
    problems = [make_problem(*s, seed=11 + i) for i, s in enumerate(shapes)]
    dev = [(a.cuda(), b.cuda()) for a, b in problems]
    outs = [torch.full((s[0], s[1]), float("nan"), dtype=torch.bfloat16, device="cuda")
            for s in shapes]
    for (M, N, K), (dA, dB), out in zip(shapes, dev, outs):
        assert _noalloc(dA, dB, out, M, N, K) == 0
        assert ops.last_config()["stream_k"] == 1
    torch.cuda.synchronize()
    assert _noalloc_status()[0] == 0
    for s, (A, B), out in zip(shapes, problems, outs):
        oracle.assert_parity(out, oracle.gemm_fp32(A, B), f"noalloc back to back {s}")


def test_noalloc_column_major_like_the_reference():
    M, N, K = 48, 2048, 1024
    A, B = make_problem(M, N, K, seed=77)
    dA, dB = A.cuda(), B.cuda()
    for _ in range(2):
        C = torch.full((N, M), float("nan"), dtype=torch.bfloat16, device="cuda")
        assert _noalloc(dA, dB, C, M, N, K, col_major=True) == 0
        assert ops.last_config()["stream_k"] == 1
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


def test_noalloc_device_error_is_visible_sticky_and_clearable():
    # The sanctioned failure: one warp waits 2 ms on a barrier nothing completes, gives up and
    # records code 4 in the entry point's own device-side word.  Nothing faults.
    M, N, K = 64, 3584, 2048
    A, B = make_problem(M, N, K, seed=3)
    dA, dB = A.cuda(), B.cuda()
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    assert _noalloc_status()[0] == 0
    assert lib.neogemm_debug_wait_expiry_noalloc(2000) == 0
    try:
        status = _noalloc_status()
        assert status[0] == 4 and status[2] == -1, status
        assert _noalloc(dA, dB, out, M, N, K) == 5          # NEOGEMM_ERR_DEVICE_TIMEOUT
        assert ops.device_status()[0] == 0                  # the regular path has its own record
    finally:
        assert lib.neogemm_noalloc_clear_status() == 0
    assert _noalloc_status() == (0, 0, 0, 0)
    out.fill_(float("nan"))
    assert _noalloc(dA, dB, out, M, N, K) == 0
    torch.cuda.synchronize()
    oracle.assert_parity(out, oracle.gemm_fp32(A, B), "noalloc after a cleared error")
