"""Seeded synthetic operands for tests and benchmarks.

The reference draws unseeded N(0,1) operands at 1024^3 (benchmark.py:10-11) and N(0,1) from
std::default_random_engine(69) in its cuBLAS harness (cublass/matmul.cu:31,53-59).  Here every
operand is N(0,1)/sqrt(K) from a seeded CPU generator, so outputs stay O(1/sqrt(K))..O(1) for any
K and every rank of a sharded run can regenerate any block from (seed, block index).
"""
from __future__ import annotations

import math

import torch

DEFAULT_SEED = 1234
ROW_BLOCK = 8192  # rows per independently seeded block of a tall operand


def make_operand(rows: int, K: int, seed: int, scale_by_k: bool = True) -> torch.Tensor:
    """bf16 [rows, K] on the CPU, N(0,1)/sqrt(K) (or N(0,1) when ``scale_by_k`` is False)."""
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    t = torch.randn(rows, K, generator=g, dtype=torch.float32)
    if scale_by_k and K > 0:
        t.mul_(1.0 / math.sqrt(K))
    return t.to(torch.bfloat16)


def make_problem(M: int, N: int, K: int, seed: int = DEFAULT_SEED, scale_by_k: bool = True):
    """(A[M,K], B[N,K]) bf16 on the CPU.  A and B come from one generator stream: A first."""
    g = torch.Generator(device="cpu").manual_seed(int(seed))
    s = 1.0 / math.sqrt(K) if (scale_by_k and K > 0) else 1.0
    A = (torch.randn(M, K, generator=g, dtype=torch.float32) * s).to(torch.bfloat16)
    B = (torch.randn(N, K, generator=g, dtype=torch.float32) * s).to(torch.bfloat16)
    return A, B


def make_row_block(block_index: int, rows: int, K: int, seed: int = DEFAULT_SEED) -> torch.Tensor:
    """Block ``block_index`` (``rows`` <= ROW_BLOCK rows) of a tall operand: seeded by
    (seed, block_index) alone so any rank can produce any block without communication."""
    return make_operand(rows, K, seed * 1_000_003 + 7919 * (block_index + 1))


def make_tall_operand(rows: int, K: int, seed: int = DEFAULT_SEED, first_row: int = 0) -> torch.Tensor:
    """Rows [first_row, first_row + rows) of the tall operand defined by make_row_block.
    ``first_row`` must be a multiple of ROW_BLOCK."""
    if first_row % ROW_BLOCK != 0:
        raise ValueError("first_row must be a multiple of ROW_BLOCK")
    out = torch.empty((rows, K), dtype=torch.bfloat16)
    r = 0
    while r < rows:
        n = min(ROW_BLOCK, rows - r)
        out[r:r + n] = make_row_block((first_row + r) // ROW_BLOCK, n, K, seed)
        r += n
    return out
