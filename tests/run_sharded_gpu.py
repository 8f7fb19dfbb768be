"""Launched by torchrun (one rank per GPU): parity of the row-sharded product on real GPUs.
Each rank builds the same seeded problem on the CPU, takes its row block of A, receives B by NCCL
broadcast (plain, chunk-overlapped and host-buffer pipeline variants) and checks its rows of C against the CPU oracle,
and B against the original bits.  Exit status 0 = every rank passed."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from gemm_b200 import ops  # noqa: E402
from gemm_b200.inputs import make_problem  # noqa: E402
from gemm_b200.shard import (row_partition, sharded_matmul, sharded_matmul_host,  # noqa: E402
                             sharded_matmul_overlapped)
from oracle import oracle  # noqa: E402


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        M, N, K = 3000, 2048, 1024
        A, B = make_problem(M, N, K, seed=2024)
        r0, r1 = row_partition(M, world, rank)
        A_block = A[r0:r1].cuda()
        B_dev = B.cuda() if rank == 0 else None
        ref = oracle.gemm_fp32(A[r0:r1], B)
        for name, fn in (("plain", sharded_matmul), ("overlapped", sharded_matmul_overlapped)):
            C_block, B_local = fn(A_block, B_dev, N, K)
            torch.cuda.synchronize()
            assert ops.device_status()[0] == 0
            assert torch.equal(B_local.cpu().view(torch.int16), B.view(torch.int16)), name
            oracle.assert_parity(C_block, ref, f"{name} rank {rank}/{world}")
        # host buffers in and out: uploads, broadcast, products and downloads overlapped
        hA = A[r0:r1].contiguous().pin_memory()
        hB = B.pin_memory() if rank == 0 else None
        hC = torch.full((r1 - r0, N), float("nan"), dtype=torch.bfloat16).pin_memory()
        for call in range(2):
            sharded_matmul_host(hA, hB, hC, N, K)
            assert ops.device_status()[0] == 0
            oracle.assert_parity(hC, ref, f"host pipeline call {call} rank {rank}/{world}")
            hC.fill_(float("nan"))
        C_full, _ = sharded_matmul(A_block, B_dev, N, K, gather=True)
        oracle.assert_parity(C_full, oracle.gemm_fp32(A, B), f"gathered rank {rank}")
        print(f"rank {rank}: sharded parity ok", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
