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
                              matmul_out: Optional[Callable] = None,
                              out: Optional[torch.Tensor] = None,
                              B_buffer: Optional[torch.Tensor] = None):
    """Same product with the broadcast of B hidden under compute: B travels in ``chunks`` row
    blocks on a side stream, and the product for the columns of C that a block feeds is launched
    as soon as that block has landed in local HBM.  The kernel still reads local memory only.

    Returns (C_block, B_local).  ``matmul_out(A, B_rows, out)`` defaults to the CUDA operator
    writing into a column slice of C (row pitch N); CPU tests inject a stand-in.  ``out`` ([rows,
    N]) and ``B_buffer`` ([N, K], used on the receiving ranks) let a caller that repeats the
    product keep its buffers instead of allocating them per call."""
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
    elif B_buffer is not None:
        if tuple(B_buffer.shape) != (N, K):
            raise ValueError(f"B_buffer must have shape [{N},{K}]")
        B_local = B_buffer
    else:
        B_local = torch.empty((N, K), dtype=A_block.dtype, device=A_block.device)
    if out is not None:
        if tuple(out.shape) != (A_block.shape[0], N):
            raise ValueError(f"out must have shape [{A_block.shape[0]},{N}]")
        C_block = out
    else:
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


class ShardedHostPipeline:
    """The sharded product for callers whose operands live in HOST memory: this rank's rows of A
    go up, its rows of C come back, and the three transfers overlap with the compute.

    Per call, on every rank:
      * the broadcasting rank uploads B in row chunks on a copy queue and hands each chunk to the
        broadcast as soon as it has landed, so the upload of chunk i+1 runs under the broadcast
        of chunk i; the other ranks only receive;
      * the A block goes up in row chunks on the same copy queue (behind B on the broadcasting
        rank, at once on the others);
      * as soon as B is complete and a chunk of A has landed, the product of that chunk is
        launched on the caller's stream, and its rows of C go back on a second copy queue while
        later chunks are still going up or being multiplied.
    Same idea as the single-GPU host entry point of the C ABI (neogemm_bf16_nt_host), extended
    by the broadcast.  The kernel reads local HBM only.  Device staging buffers and streams are
    created once and reused; one call at a time per pipeline.  Host tensors should be pinned,
    otherwise the copies serialise.  On CPU tensors (tests of the host logic on gloo ranks) the
    same sequence runs without streams and with an injected product."""

    def __init__(self, rows: int, N: int, K: int, device, group=None, src: int = 0,
                 row_chunks: int = 0, b_chunks: int = 4, matmul_out: Optional[Callable] = None,
                 dtype=torch.bfloat16):
        self.rows, self.N, self.K = int(rows), int(N), int(K)
        self.device = torch.device(device)
        self.group, self.src = group, src
        self.on_gpu = self.device.type == "cuda"
        if matmul_out is None:
            from .ops import matmul as _mm

            def matmul_out(a, b, out):  # noqa: ANN001
                _mm(a, b, out=out)
        self.matmul_out = matmul_out
        # Row chunks of A on multiples of 256 rows (whole tiles), at least 1024 rows each so that
        # every launch still fills the GPU, at most 16 chunks.
        if row_chunks <= 0:
            row_chunks = max(1, min(16, self.rows // 1024))
        per = ((self.rows + row_chunks - 1) // row_chunks + 255) // 256 * 256 if self.rows else 0
        self.a_bounds = [(r, min(r + per, self.rows)) for r in range(0, self.rows, per)] if per else []
        b_chunks = max(1, min(b_chunks, (self.N + 255) // 256))
        perb = ((self.N + b_chunks - 1) // b_chunks + 255) // 256 * 256
        self.b_bounds = [(n, min(n + perb, self.N)) for n in range(0, self.N, perb)]
        self.dA = torch.empty((self.rows, self.K), dtype=dtype, device=self.device)
        self.dB = torch.empty((self.N, self.K), dtype=dtype, device=self.device)
        self.dC = torch.empty((self.rows, self.N), dtype=dtype, device=self.device)
        if self.on_gpu:
            self.s_in = torch.cuda.Stream(device=self.device)
            self.s_out = torch.cuda.Stream(device=self.device)
            self.s_comm = torch.cuda.Stream(device=self.device)

    def h2d_bytes(self, rank: int) -> int:
        es = self.dA.element_size()
        return self.rows * self.K * es + (self.N * self.K * es if rank == self.src else 0)

    def d2h_bytes(self) -> int:
        return self.rows * self.N * self.dC.element_size()

    def run(self, hA_block: torch.Tensor, hB: Optional[torch.Tensor], hC_block: torch.Tensor,
            wait: bool = True) -> torch.Tensor:
        import torch.distributed as dist
        rank = dist.get_rank(self.group)
        if tuple(hA_block.shape) != (self.rows, self.K) or tuple(hC_block.shape) != (self.rows, self.N):
            raise ValueError("host blocks do not match the pipeline's shape")
        if rank == self.src and (hB is None or tuple(hB.shape) != (self.N, self.K)):
            raise ValueError(f"rank {self.src} must supply B with shape [{self.N},{self.K}]")
        if not self.on_gpu:
            for n0, n1 in self.b_bounds:
                if rank == self.src:
                    self.dB[n0:n1].copy_(hB[n0:n1])
                dist.broadcast(self.dB[n0:n1], src=self.src, group=self.group)
            for r0, r1 in self.a_bounds:
                self.dA[r0:r1].copy_(hA_block[r0:r1])
                self.matmul_out(self.dA[r0:r1], self.dB, self.dC[r0:r1])
                hC_block[r0:r1].copy_(self.dC[r0:r1])
            return hC_block
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_out, self.s_comm):
            s.wait_stream(cur)
        # B: upload (broadcasting rank) chunk by chunk, each chunk broadcast as it lands.
        for n0, n1 in self.b_bounds:
            if rank == self.src:
                with torch.cuda.stream(self.s_in):
                    self.dB[n0:n1].copy_(hB[n0:n1], non_blocking=True)
                    landed = torch.cuda.Event()
                    landed.record(self.s_in)
                self.s_comm.wait_event(landed)
            with torch.cuda.stream(self.s_comm):
                dist.broadcast(self.dB[n0:n1], src=self.src, group=self.group)
        b_ready = torch.cuda.Event()
        b_ready.record(self.s_comm)
        # A: row chunks up; product per landed chunk; rows of C down.
        ups = []
        with torch.cuda.stream(self.s_in):
            for r0, r1 in self.a_bounds:
                self.dA[r0:r1].copy_(hA_block[r0:r1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self.s_in)
                ups.append(ev)
        cur.wait_event(b_ready)
        for i, ((r0, r1), up) in enumerate(zip(self.a_bounds, ups)):
            cur.wait_event(up)
            self.matmul_out(self.dA[r0:r1], self.dB, self.dC[r0:r1])
            done = torch.cuda.Event()
            done.record(cur)
            self.s_out.wait_event(done)
            # Downloads start on upload boundaries (a download that starts in the middle of an
            # upload slows it by more than the wait costs: measured on the single-GPU entry point).
            if i + 1 < len(ups):
                self.s_out.wait_event(ups[i + 1])
            with torch.cuda.stream(self.s_out):
                hC_block[r0:r1].copy_(self.dC[r0:r1], non_blocking=True)
        cur.wait_stream(self.s_out)
        if wait:
            self.s_out.synchronize()
        return hC_block


_host_pipelines = {}


def sharded_matmul_host(hA_block: torch.Tensor, hB: Optional[torch.Tensor], hC_block: torch.Tensor,
                        N: int, K: int, device=None, group=None, src: int = 0,
                        matmul_out: Optional[Callable] = None) -> torch.Tensor:
    """C_block (host) = A_block (host) * B^T with B (host, on rank ``src`` only) broadcast over
    NCCL: uploads, broadcast, products and downloads overlapped (see ShardedHostPipeline).
    Returns ``hC_block`` once its contents are complete."""
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")
    key = (int(hA_block.shape[0]), int(N), int(K), str(device), id(group), src, hA_block.dtype)
    pipe = _host_pipelines.get(key)
    if pipe is None or matmul_out is not None:
        pipe = ShardedHostPipeline(hA_block.shape[0], N, K, device, group=group, src=src,
                                   matmul_out=matmul_out, dtype=hA_block.dtype)
        if matmul_out is None:
            _host_pipelines.clear()   # one resident set of staging buffers
            _host_pipelines[key] = pipe
    return pipe.run(hA_block, hB, hC_block)
