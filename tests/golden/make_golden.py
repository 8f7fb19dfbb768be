"""Generates the committed fixtures gemm_*.npz: seeded bf16 operands (bit patterns) and the
scalar C oracle's bf16 result (bit patterns, row-major [M,N]).

The reference has no fixtures of its own and cannot be run, so these freeze the oracle's output
rather than the reference's.  Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from gemm_b200.inputs import make_problem  # noqa: E402
from oracle import oracle  # noqa: E402

CASES = [  # (M, N, K, seed): aligned, ragged M/N, ragged K (K % 64 != 0), skinny
    (64, 64, 64, 101),
    (128, 256, 128, 102),
    (100, 72, 200, 103),
    (16, 384, 512, 104),
    (130, 33, 72, 105),
]

if __name__ == "__main__":
    here = os.path.dirname(os.path.abspath(__file__))
    for M, N, K, seed in CASES:
        A, B = make_problem(M, N, K, seed=seed)
        C = oracle.gemm_scalar_c(A, B)
        np.savez_compressed(
            os.path.join(here, f"gemm_{M}x{N}x{K}_s{seed}.npz"),
            M=M, N=N, K=K, seed=seed,
            A_bits=A.view(torch.int16).numpy(), B_bits=B.view(torch.int16).numpy(),
            C_bits=C.view(torch.int16).numpy())
        print("wrote", M, N, K, seed)
