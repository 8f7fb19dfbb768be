"""CPU: the oracle's three restatements agree with each other and with the committed fixtures."""
import glob
import os

import numpy as np
import pytest
import torch

from gemm_b200.inputs import make_problem
from oracle import oracle

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("shape", [(1, 1, 8), (7, 5, 16), (64, 64, 64), (96, 80, 136), (130, 33, 264)])
def test_scalar_loop_matches_fp64_and_torch(shape):
    M, N, K = shape
    A, B = make_problem(M, N, K, seed=11)
    f64 = oracle.gemm_f64(A, B)
    ref = oracle.gemm_fp32(A, B)
    # fp32 accumulation error over K terms of magnitude ~1/K each
    assert (ref.double() - f64).abs().max() < 1e-5
    c = oracle.gemm_scalar_c(A, B)
    s = oracle.compare(c, ref)
    assert s["max_ulp"] <= 1 and s["bit_equal_frac"] > 0.99, s
    # and against exact arithmetic rounded once
    s64 = oracle.compare(c, f64.float())
    assert s64["max_ulp"] <= 1 and s64["near_zero_ok"], s64


def test_column_major_is_the_transpose():
    A, B = make_problem(40, 24, 64, seed=3)
    row = oracle.gemm_scalar_c(A, B, col_major=False)
    col = oracle.gemm_scalar_c(A, B, col_major=True)
    assert col.shape == (24, 40)
    assert torch.equal(col.t().contiguous().view(torch.int16), row.view(torch.int16))
    assert torch.equal(oracle.gemm_bf16(A, B, col_major=True).view(torch.int16),
                       oracle.gemm_bf16(A, B).t().contiguous().view(torch.int16))


def test_round_to_nearest_even_rule():
    c = oracle._c()
    # exactly representable
    assert c.oracle_f32_to_bf16(1.0) == 0x3F80
    # 1 + 2^-8 is a tie between 0x3F80 and 0x3F81 -> even (0x3F80)
    assert c.oracle_f32_to_bf16(1.0 + 2.0 ** -8) == 0x3F80
    # 1 + 3*2^-8 is a tie between 0x3F81 and 0x3F82 -> even (0x3F82)
    assert c.oracle_f32_to_bf16(1.0 + 3 * 2.0 ** -8) == 0x3F82
    # just above the tie rounds up
    assert c.oracle_f32_to_bf16(1.0 + 2.0 ** -8 + 2.0 ** -20) == 0x3F81
    assert c.oracle_f32_to_bf16(-2.5) == 0xC020
    # agrees with torch's conversion on random values
    x = torch.randn(4096, generator=torch.Generator().manual_seed(5))
    mine = torch.tensor([c.oracle_f32_to_bf16(float(v)) for v in x], dtype=torch.int32)
    theirs = x.to(torch.bfloat16).view(torch.int16).to(torch.int32) & 0xFFFF
    assert torch.equal(mine, theirs)


def test_unscaled_inputs_like_the_reference_driver():
    # benchmark.py:10-11 uses unscaled N(0,1); outputs are O(sqrt(K)).
    A, B = make_problem(32, 48, 256, seed=9, scale_by_k=False)
    ref = oracle.gemm_fp32(A, B)
    c = oracle.gemm_scalar_c(A, B)
    assert oracle.compare(c, ref)["max_ulp"] <= 1
    assert ref.abs().max() > 10


def test_golden_fixtures():
    files = sorted(glob.glob(os.path.join(GOLDEN, "gemm_*.npz")))
    assert len(files) >= 4, "fixtures missing: run tests/golden/make_golden.py"
    for f in files:
        z = np.load(f)
        M, N, K, seed = (int(z[k]) for k in ("M", "N", "K", "seed"))
        A, B = make_problem(M, N, K, seed=seed)
        assert np.array_equal(A.view(torch.int16).numpy(), z["A_bits"]), f
        assert np.array_equal(B.view(torch.int16).numpy(), z["B_bits"]), f
        c = oracle.gemm_scalar_c(A, B)
        assert np.array_equal(c.view(torch.int16).numpy(), z["C_bits"]), f
        ref = oracle.gemm_fp32(A, B)
        s = oracle.compare(torch.from_numpy(z["C_bits"]).view(torch.bfloat16), ref)
        assert s["max_ulp"] <= 1 and s["allclose_1e-2"], (f, s)
