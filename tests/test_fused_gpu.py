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
    (64, 28672, 1024), (24, 20000, 1024),
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
