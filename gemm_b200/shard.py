"""Row-sharded GEMM over the GPUs of one node: C[M,N] = A[M,K] * B[N,K]^T with A split into
contiguous row blocks, one per rank; B is broadcast once; no reduction follows because rows of C
depend only on the same rows of A.

The reference is single-GPU (no NCCL, MPI or torch.distributed call in any of its files); this is
the data-parallel extension of its operator.  Each rank's kernel reads only its own GPU's memory:
the broadcast lands B in local HBM first.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch


def row_partition(M: int, world: int, rank: int, align: int = 128) -> Tuple[int, int]:
    """Rows [r0, r1) of A (and of C) owned by ``rank``.  Blocks are contiguous, cover [0, M)
    exactly, differ by less than two ``align`` units, and start on multiples of ``align`` (one tensor-core
    tile) so no tile straddles two ranks."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if M < 0:
        raise ValueError("M must be non-negative")
    units = (M + align - 1) // align
    base, extra = divmod(units, world)
    u0 = rank * base + min(rank, extra)
    u1 = u0 + base + (1 if rank < extra else 0)
    return min(u0 * align, M), min(u1 * align, M)


def sharded_matmul(A_block: torch.Tensor, B: Optional[torch.Tensor], N: int, K: int,
                   group=None, src: int = 0,
                   matmul: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None,
                   gather: bool = False):
    """One sharded product.  ``A_block`` is this rank's rows of A; ``B`` is the full [N,K] operand
    on rank ``src`` (ignored, may be None, elsewhere).  Returns (C_block, B_local) or, with
    ``gather``, (C_full on every rank, B_local).

    ``matmul`` defaults to the CUDA operator; tests of the host-side logic on CPU ranks inject a
    stand-in (the library itself has no CPU path)."""
    import torch.distributed as dist
    if matmul is None:
        from .ops import matmul as matmul  # noqa: PLW0127
    rank = dist.get_rank(group)
    if rank == src:
        if B is None or tuple(B.shape) != (N, K):
            raise ValueError(f"rank {src} must supply B with shape [{N},{K}]")
        B_local = B
    else:
        B_local = torch.empty((N, K), dtype=A_block.dtype, device=A_block.device)
    dist.broadcast(B_local, src=src, group=group)
    C_block = matmul(A_block, B_local)
    if not gather:
        return C_block, B_local
    world = dist.get_world_size(group)
    sizes = torch.zeros(world, dtype=torch.int64, device=A_block.device)
    sizes[rank] = C_block.shape[0]
    dist.all_reduce(sizes, group=group)
    # all_gather wants equal shapes: pad every block to the tallest one, trim afterwards.
    tallest = int(sizes.max())
    padded = torch.zeros((tallest, N), dtype=C_block.dtype, device=C_block.device)
    padded[:C_block.shape[0]] = C_block
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded, group=group)
    return torch.cat([p[:int(n)] for p, n in zip(parts, sizes)], dim=0), B_local


def sharded_matmul_overlapped(A_block: torch.Tensor, B: Optional[torch.Tensor], N: int, K: int,
                              chunks: int = 4, group=None, src: int = 0,
                              matmul_out: Optional[Callable] = None):
    """Same product with the broadcast of B hidden under compute: B travels in ``chunks`` row
    blocks on a side stream, and the product for the columns of C that a block feeds is launched
    as soon as that block has landed in local HBM.  The kernel still reads local memory only.

    Returns (C_block, B_local).  ``matmul_out(A, B_rows, out)`` defaults to the CUDA operator
    writing into a column slice of C (row pitch N); CPU tests inject a stand-in."""
    import torch.distributed as dist
    if matmul_out is None:
        from .ops import matmul as _mm

        def matmul_out(a, b, out):  # noqa: ANN001
            _mm(a, b, out=out)
    rank = dist.get_rank(group)
    if rank == src:
        if B is None or tuple(B.shape) != (N, K):
            raise ValueError(f"rank {src} must supply B with shape [{N},{K}]")
        B_local = B
    else:
        B_local = torch.empty((N, K), dtype=A_block.dtype, device=A_block.device)
    C_block = torch.empty((A_block.shape[0], N), dtype=A_block.dtype, device=A_block.device)
    # Column blocks on multiples of 256 (one tile) so that every launch sees whole tiles.
    chunks = max(1, min(chunks, (N + 255) // 256))
    per = ((N + chunks - 1) // chunks + 255) // 256 * 256
    bounds = [(n0, min(n0 + per, N)) for n0 in range(0, N, per)]
    on_gpu = A_block.is_cuda
    if on_gpu:
        compute = torch.cuda.current_stream(A_block.device)
        side = torch.cuda.Stream(device=A_block.device)
        side.wait_stream(compute)
        events = []
        with torch.cuda.stream(side):
            for n0, n1 in bounds:
                dist.broadcast(B_local[n0:n1], src=src, group=group)
                ev = torch.cuda.Event()
                ev.record(side)
                events.append(ev)
        for (n0, n1), ev in zip(bounds, events):
            compute.wait_event(ev)
            matmul_out(A_block, B_local[n0:n1], C_block[:, n0:n1])
        B_local.record_stream(side)
    else:
        for n0, n1 in bounds:
            dist.broadcast(B_local[n0:n1], src=src, group=group)
            matmul_out(A_block, B_local[n0:n1], C_block[:, n0:n1])
    return C_block, B_local
