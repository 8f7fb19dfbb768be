"""GPU parity of the fused epilogue: C = act(alpha * A B^T + beta * C + bias), checked against the
same formula applied in fp32 to the CPU oracle's unrounded product."""
import math

import pytest
import torch

from gemm_b200 import ops
from gemm_b200.inputs import make_problem
from oracle import oracle

pytestmark = pytest.mark.gpu


def reference(A, B, alpha, beta, c_old, bias, activation):
    v = alpha * oracle.gemm_fp32(A, B)
    if beta != 0.0:
        v = v + beta * c_old.float()
    if bias is not None:
        v = v + bias.float()[None, :]
    if activation == "relu":
        v = torch.relu(v)
    elif activation == "gelu_tanh":
        v = torch.nn.functional.gelu(v, approximate="tanh")
    return v


CASES = [  # (M, N, K): pair kernel, cut last wave, single-CTA TMA store, direct, swapped stream-K,
    # whole tiles two CTAs to an SM
    (2048, 2048, 512), (4096, 4096, 1024), (520, 776, 264), (257, 250, 128), (16, 3584, 2048),
    (64, 28672, 1024), (24, 20000, 1024), (1024, 1024, 4096),   # the last: two-pass split-K
    (128, 28672, 1024),   # tall pair tiles of 128 columns: fused calls keep the usual operand roles
]


@pytest.mark.parametrize("shape", CASES)
@pytest.mark.parametrize("activation", ["none", "relu", "gelu_tanh"])
def test_alpha_beta_bias_activation(shape, activation):
    M, N, K = shape
    A, B = make_problem(M, N, K, seed=M + N + K)
    g = torch.Generator().manual_seed(3)
    c_old = (torch.randn(M, N, generator=g) * 0.05).to(torch.bfloat16)
    bias = (torch.randn(N, generator=g) * 0.05).to(torch.bfloat16)
    alpha, beta = 0.75, -0.5
    out = c_old.cuda()
    ops.matmul_fused(A.cuda(), B.cuda(), out=out, alpha=alpha, beta=beta, bias=bias.cuda(),
                     activation=activation)
    cfg = ops.last_config()
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    want = reference(A, B, alpha, beta, c_old, bias, activation)
    # tanhf on the device and torch's CPU tanh may differ in the last fp32 bits, which can move a
    # bf16 rounding: allow 2 ulp for GELU, 1 otherwise.
    oracle.assert_parity(out, want, f"fused {shape} {activation} cfg={cfg}",
                         max_ulp=2 if activation == "gelu_tanh" else 1, bit_equal=0.97)


def test_fusion_defaults_equal_the_plain_product():
    A, B = make_problem(1024, 768, 512, seed=8)
    dA, dB = A.cuda(), B.cuda()
    plain = ops.matmul(dA, dB)
    fused = ops.matmul_fused(dA, dB)
    assert torch.equal(plain.view(torch.int16), fused.view(torch.int16))


def test_column_major_bias_runs_along_n():
    M, N, K = 384, 640, 256
    A, B = make_problem(M, N, K, seed=10)
    bias = (torch.randn(N, generator=torch.Generator().manual_seed(1)) * 0.1).to(torch.bfloat16)
    out = ops.matmul_fused(A.cuda(), B.cuda(), bias=bias.cuda(), col_major=True)
    assert out.shape == (N, M)
    want = reference(A, B, 1.0, 0.0, None, bias, "none")
    oracle.assert_parity(out.t(), want, "fused column-major bias")


def test_bad_fusion_arguments():
    A, B = make_problem(64, 64, 64, seed=1)
    with pytest.raises(ValueError):
        ops.matmul_fused(A.cuda(), B.cuda(), beta=1.0)
    with pytest.raises(ValueError):
        ops.matmul_fused(A.cuda(), B.cuda(), activation="swish")
    with pytest.raises(ValueError):
        ops.matmul_fused(A.cuda(), B.cuda(), bias=torch.zeros(3, dtype=torch.bfloat16, device="cuda"))


# ---- fp32 result ---------------------------------------------------------------------------------
def assert_fp32_result(out, want, what):
    """Gates for an UNROUNDED result: what separates the kernel's fp32 accumulator from the CPU's
    is summation order only, so the error must sit far below one bf16 rounding (relative
    Frobenius 1.7e-3, which is what a result rounded to bf16 on the way would show)."""
    assert out.dtype == torch.float32
    o = out.detach().cpu().double()
    w = want.double()
    assert bool(torch.isfinite(o).all()), f"{what}: non-finite or unwritten (NaN-poisoned) elements"
    rms = float(w.pow(2).mean().sqrt())
    rel_fro = float(torch.linalg.norm(o - w) / torch.linalg.norm(w))
    max_abs = float((o - w).abs().max())
    assert rel_fro <= 1e-4, f"{what}: relative Frobenius error {rel_fro:.3e}"
    assert max_abs <= 1e-3 * rms, f"{what}: max |error| {max_abs:.3e} against rms {rms:.3e}"
    return {"rel_fro": rel_fro, "max_abs": max_abs, "rms": rms}


F32_CASES = [  # pair TMA-store, cut last wave, single-CTA TMA store, ragged edges with TMA store,
    # direct (N % 4 != 0), swapped stream-K, swapped whole tiles two CTAs to an SM, data-parallel
    (2048, 2048, 512), (4096, 4096, 1024), (520, 776, 264), (1000, 1004, 520), (257, 250, 128),
    (16, 3584, 2048), (64, 28672, 1024), (1024, 768, 512), (1024, 1024, 4096),
]


@pytest.mark.parametrize("shape", F32_CASES)
def test_fp32_result_plain_and_fused(shape):
    M, N, K = shape
    A, B = make_problem(M, N, K, seed=M + 2 * N + K)
    dA, dB = A.cuda(), B.cuda()
    ref = oracle.gemm_fp32(A, B)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device="cuda")
    ops.matmul_fused(dA, dB, out=out)
    cfg = ops.last_config()
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    stats = assert_fp32_result(out, ref, f"fp32 result {shape} cfg={cfg}")
    assert cfg["block_n"] <= 256, cfg   # never the two-half tile
    # The same product rounded once must be the bf16 entry point's result, bit for bit - with K
    # walked forwards by every tile in both: the bf16 entry point may pick a different tile (and
    # so different waves), and by default the K direction alternates from wave to wave.
    ops.set_tuning("k_direction_alternates", 0)
    try:
        fwd32 = ops.matmul_fused(dA, dB, out_dtype=torch.float32)
        fwd16 = ops.matmul(dA, dB)
    finally:
        ops.set_tuning("k_direction_alternates", -1)
    assert torch.equal(fwd32.to(torch.bfloat16).view(torch.int16), fwd16.view(torch.int16)), \
        (shape, cfg, stats)
    # alpha, beta (read as fp32), bias and activation on top
    g = torch.Generator().manual_seed(5)
    c_old = torch.randn(M, N, generator=g) * 0.05
    bias = (torch.randn(N, generator=g) * 0.05).to(torch.bfloat16)
    out = c_old.cuda()
    ops.matmul_fused(dA, dB, out=out, alpha=1.25, beta=0.5, bias=bias.cuda(), activation="relu")
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    want = torch.relu(1.25 * ref + 0.5 * c_old + bias.float()[None, :])
    assert_fp32_result(out, want, f"fp32 fused {shape}")


def test_fp32_result_column_major_and_pitch():
    M, N, K = 384, 640, 256
    A, B = make_problem(M, N, K, seed=12)
    ref = oracle.gemm_fp32(A, B)
    out = ops.matmul_fused(A.cuda(), B.cuda(), col_major=True, out_dtype=torch.float32)
    assert out.shape == (N, M) and out.dtype == torch.float32
    assert_fp32_result(out.t(), ref, "fp32 column-major")
    # a padded row pitch (ldc = N + 4 floats: still 16-byte rows) and an odd one (direct stores)
    for pad in (4, 3):
        wide = torch.full((M, N + pad), float("nan"), dtype=torch.float32, device="cuda")
        view = wide[:, :N]
        ops.matmul_fused(A.cuda(), B.cuda(), out=view)
        torch.cuda.synchronize()
        assert_fp32_result(view, ref, f"fp32 pitch N+{pad}")
        assert bool(torch.isnan(wide[:, N:]).all()), "wrote outside the result's columns"
