"""CPU: partition arithmetic and the sharded-GEMM host logic on two gloo ranks.  The per-rank
product is a stand-in (the oracle) because the library has no CPU path; what is under test is
the partition, the broadcast of B and the gather."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from gemm_b200.shard import row_partition


@pytest.mark.parametrize("M", [0, 1, 127, 128, 129, 1000, 8192, 131072, 131073])
@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_partition_covers_rows_exactly(M, world):
    edges = [row_partition(M, world, r) for r in range(world)]
    assert edges[0][0] == 0 and edges[-1][1] == M
    for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
        assert a1 == b0 and a0 <= a1
    sizes = [b - a for a, b in edges]
    assert max(sizes) - min(sizes) < 256 or M < 128 * world
    for a, b in edges[:-1]:
        assert a % 128 == 0 or a == M


def test_partition_of_the_benchmark_shape():
    for world, rows in ((1, 131072), (2, 65536), (4, 32768), (8, 16384)):
        for r in range(world):
            assert row_partition(131072, world, r) == (r * rows, (r + 1) * rows)


def test_partition_rejects_bad_rank():
    with pytest.raises(ValueError):
        row_partition(10, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, out_dir):
    import torch.distributed as dist
    from gemm_b200.inputs import make_problem
    from gemm_b200.shard import row_partition, sharded_matmul
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        A, B = make_problem(M, N, K, seed=99)
        r0, r1 = row_partition(M, world, rank)
        stand_in = lambda a, b: oracle.gemm_bf16(a, b)  # noqa: E731
        C_full, B_local = sharded_matmul(A[r0:r1].contiguous(), B if rank == 0 else None, N, K,
                                         matmul=stand_in, gather=True)
        assert torch.equal(B_local.view(torch.int16), B.view(torch.int16)), "broadcast of B"
        want = oracle.gemm_bf16(A, B)
        assert torch.equal(C_full.view(torch.int16), want.view(torch.int16)), "gathered C"
        C_block, _ = sharded_matmul(A[r0:r1].contiguous(), B if rank == 0 else None, N, K,
                                    matmul=stand_in)
        assert C_block.shape == (r1 - r0, N)
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_sharded_product_on_two_gloo_ranks(tmp_path):
    world = 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, 300, 72, 64, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_rank_zero_must_supply_b(tmp_path):
    # Host-side failure: detected before any collective is issued.
    import torch.distributed as dist
    from gemm_b200.shard import sharded_matmul
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(_free_port())
    dist.init_process_group("gloo", rank=0, world_size=1)
    try:
        with pytest.raises(ValueError):
            sharded_matmul(torch.zeros(4, 8, dtype=torch.bfloat16), None, 6, 8,
                           matmul=lambda a, b: a.float() @ b.float().t())
    finally:
        dist.destroy_process_group()


def _worker_overlap(rank, world, port, M, N, K, out_dir):
    import torch.distributed as dist
    from gemm_b200.inputs import make_problem
    from gemm_b200.shard import row_partition, sharded_matmul_overlapped
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        A, B = make_problem(M, N, K, seed=5)
        r0, r1 = row_partition(M, world, rank)

        def stand_in(a, b, out):
            out.copy_(oracle.gemm_bf16(a, b.contiguous()))
        C_block, B_local = sharded_matmul_overlapped(A[r0:r1].contiguous(), B if rank == 0 else None,
                                                     N, K, chunks=3, matmul_out=stand_in)
        assert torch.equal(B_local.view(torch.int16), B.view(torch.int16))
        want = oracle.gemm_bf16(A, B)[r0:r1]
        assert torch.equal(C_block.view(torch.int16), want.contiguous().view(torch.int16))
        # with the caller's buffers
        keep_c = torch.full((r1 - r0, N), float("nan"), dtype=torch.bfloat16)
        keep_b = B.clone() if rank == 0 else torch.zeros((N, K), dtype=torch.bfloat16)
        C2, B2 = sharded_matmul_overlapped(A[r0:r1].contiguous(), keep_b if rank == 0 else None, N, K,
                                           chunks=2, matmul_out=stand_in, out=keep_c,
                                           B_buffer=keep_b)
        assert C2 is keep_c and (rank == 0 or B2 is keep_b)
        assert torch.equal(keep_b.view(torch.int16), B.view(torch.int16))
        assert torch.equal(keep_c.view(torch.int16), want.contiguous().view(torch.int16))
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_overlapped_broadcast_on_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_worker_overlap, args=(world, _free_port(), 200, 700, 64, str(tmp_path)),
             nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def _worker_host_pipeline(rank, world, port, M, N, K, out_dir):
    import torch.distributed as dist
    from gemm_b200.inputs import make_problem
    from gemm_b200.shard import ShardedHostPipeline, row_partition, sharded_matmul_host
    from oracle import oracle
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        A, B = make_problem(M, N, K, seed=8)
        r0, r1 = row_partition(M, world, rank)
        calls = []

        def stand_in(a, b, out):
            calls.append(tuple(a.shape))
            out.copy_(oracle.gemm_bf16(a.contiguous(), b.contiguous()))
        hC = torch.full((r1 - r0, N), float("nan"), dtype=torch.bfloat16)
        sharded_matmul_host(A[r0:r1].contiguous(), B if rank == 0 else None, hC, N, K,
                            device="cpu", matmul_out=stand_in)
        want = oracle.gemm_bf16(A, B)[r0:r1].contiguous()
        assert torch.equal(hC.view(torch.int16), want.view(torch.int16)), "host pipeline rows of C"
        # explicit chunking: three row chunks on 256-row boundaries, two chunks of B
        pipe = ShardedHostPipeline(r1 - r0, N, K, "cpu", row_chunks=3, b_chunks=2,
                                   matmul_out=stand_in)
        assert all(a % 256 == 0 for a, _ in pipe.a_bounds) and pipe.a_bounds[-1][1] == r1 - r0
        assert pipe.b_bounds[0][0] == 0 and pipe.b_bounds[-1][1] == N
        calls.clear()
        hC.fill_(float("nan"))
        pipe.run(A[r0:r1].contiguous(), B if rank == 0 else None, hC)
        assert len(calls) == len(pipe.a_bounds) and sum(c[0] for c in calls) == r1 - r0
        assert torch.equal(hC.view(torch.int16), want.view(torch.int16))
        assert torch.equal(pipe.dB.view(torch.int16), B.view(torch.int16)), "broadcast of B"
        assert pipe.h2d_bytes(rank) == (r1 - r0) * K * 2 + (N * K * 2 if rank == 0 else 0)
        if rank == 0:
            with pytest.raises(ValueError):
                pipe.run(A[r0:r1].contiguous(), None, hC)
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(180)
def test_host_pipeline_on_two_gloo_ranks(tmp_path):
    world = 2
    mp.spawn(_worker_host_pipeline, args=(world, _free_port(), 1500, 520, 64, str(tmp_path)),
             nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


@pytest.mark.gpu
@pytest.mark.timeout(600)
def test_sharded_product_on_the_gpus_of_this_box():
    """One process per GPU over NCCL (needs at least two GPUs; skipped on a single-GPU box)."""
    import subprocess
    import sys
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    world = 2 if n < 4 else 4
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(root, "tests", "run_sharded_gpu.py")]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=540, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    assert out.stdout.count("sharded parity ok") == world
