#!/usr/bin/env python
"""Benchmark of the BF16 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the hot path over one batch of synthetic operands: one GEMM launch per
GPU.  N = 1 runs the headline 8192^3 shape; N > 1 (launched by torchrun, one rank per GPU) runs
the row-sharded 131072 x 8192 x 8192 GEMM: A is split into N contiguous row blocks, B is broadcast
once from rank 0 with NCCL (timed separately), no reduction follows.  Rank 0 prints one JSON line.

`value` is device-timed (CUDA events on the launching stream, max over ranks) with operands
resident in HBM.  `e2e` is the same metric through the C ABI's host entry point with pinned HOST
buffers: host->device copies of A and B and the device->host copy of C are inside the timed region.
`--impl reference` times the CPU restatement of the path (oracle/oracle.py: torch fp32 matmul on
all host cores) - the reference has no CPU implementation and its GPU kernels cannot run on sm_100.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "bf16_gemm_tflops"
UNIT = "TFLOP/s"

WORKLOADS = {
    # name: (M, N, K) on ONE GPU
    "8192": (8192, 8192, 8192),
    "4096": (4096, 4096, 4096),
    "512": (512, 512, 512),
    "decode16": (16, 28672, 8192),
    "decode64": (64, 28672, 8192),
    "decode128": (128, 28672, 8192),
    "sharded": (131072, 8192, 8192),   # total M; split over the ranks
}


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the dominant kernel,
# from the ncu captures summarised under profiles/ (same bench.py command lines).
NCU_TRAFFIC_BYTES = {
    "8192": 835020800 + 140674560,
    "decode16": 470125312 + 3457792,
    "decode128": 472712704 + 3770624,
}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="auto", choices=["auto"] + list(WORKLOADS))
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-cublas", action="store_true")
    ap.add_argument("--override", default="",
                    help="tuning only: kernel override, e.g. cta_group=2,block_n=256,group_m=8")
    return ap.parse_args()


def workload_for(args):
    name = args.workload
    if name == "auto":
        name = "8192" if args.gpus == 1 else "sharded"
    return name, WORKLOADS[name]


# ---------------------------------------------------------------------------------------------
# clocks
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with NVML while a region runs."""

    REASONS = {
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000080: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            self._nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in self.REASONS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def __enter__(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def record(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# reference arm: the CPU restatement of the path on the host cores
# ---------------------------------------------------------------------------------------------
def cpu_sample_rows(M):
    return min(M, 2048)


def time_cpu_oracle(M, N, K, seed, steps, warmup):
    """Times oracle.gemm_fp32 on a bounded sample: the first min(M, 2048) rows of A against all
    of B (same flops per row as the full workload)."""
    from gemm_b200.inputs import make_operand
    from oracle import oracle
    rows = cpu_sample_rows(M)
    A = make_operand(rows, K, seed)
    B = make_operand(N, K, seed + 1)
    for _ in range(warmup):
        oracle.gemm_fp32(A, B)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.gemm_fp32(A, B)
    dt = (time.perf_counter() - t0) / max(steps, 1)
    return 2.0 * rows * N * K / dt / 1e12, dt, rows


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins OMP_NUM_THREADS=1 for its ranks; the CPU arm is meant to use every host core.
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    name, (M, N, K) = workload_for(args)
    m_rank = M // args.gpus if name == "sharded" else M
    steps = max(1, min(args.steps, 20))
    warmup = max(1, min(args.warmup, 3))
    tflops, dt, rows = time_cpu_oracle(m_rank, N, K, args.seed, steps, warmup)
    cores = torch.get_num_threads()
    sample = (f"first {rows} of {m_rank} rows of A x all {N} rows of B, K={K}, "
              f"torch CPU fp32 matmul of the bf16 operands, {steps} steps")
    line = {
        "impl": "reference", "metric": METRIC, "value": tflops, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if name == "sharded" else "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": {"workload": workload_label(name, M, N, K, args.gpus)},
        "cpu_baseline": {"value": tflops, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": tflops, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_label(name, M, N, K, gpus):
    if name == "sharded":
        return (f"bf16 GEMM C=A*B^T M={M} N={N} K={K}, A row-sharded over {gpus} GPU(s) "
                f"({M // gpus} rows each), B broadcast once, N(0,1)/sqrt(K) seeded operands")
    return f"bf16 GEMM C=A*B^T M={M} N={N} K={K}, fp32 accumulate, N(0,1)/sqrt(K) seeded operands"


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def device_operand(rows, K, seed, device):
    """Operands are generated on the device for speed at the large sizes (the timing does not
    depend on values); parity is the tests' job and uses the CPU-seeded generator."""
    g = torch.Generator(device=device).manual_seed(seed)
    out = torch.empty((rows, K), dtype=torch.bfloat16, device=device)
    step = 16384
    for r in range(0, rows, step):
        n = min(step, rows - r)
        out[r:r + n] = (torch.randn(n, K, generator=g, device=device) / (K ** 0.5)).to(torch.bfloat16)
    return out


def time_launches(fn, steps, stream):
    start = torch.cuda.Event(enable_timing=True)
    stop = torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop) / 1e3   # seconds


def run_ours(args):
    from gemm_b200 import ops, roofline
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit(f"--gpus {args.gpus} needs torchrun with {args.gpus} ranks")
        raise SystemExit(f"WORLD_SIZE={world} does not match --gpus {args.gpus}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    name, (M, N, K) = workload_for(args)
    if name == "sharded":
        from gemm_b200.shard import row_partition
        r0, r1 = row_partition(M, world, rank)
        m_rank = r1 - r0
    else:
        m_rank = M
    stream = torch.cuda.current_stream(device)

    # ---- operands resident in HBM -----------------------------------------------------------
    A = device_operand(m_rank, K, args.seed + 17 * (rank + 1), device)
    bcast_ms = None
    if world > 1:
        B = device_operand(N, K, args.seed, device) if rank == 0 else \
            torch.empty((N, K), dtype=torch.bfloat16, device=device)
        dist.broadcast(B, src=0)          # warm-up of the communicator
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        dist.broadcast(B, src=0)
        e1.record()
        e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        bcast_ms = float(t.item())
    else:
        B = device_operand(N, K, args.seed, device)
    C = torch.empty((m_rank, N), dtype=torch.bfloat16, device=device)

    if args.override:
        ops.set_override(**{k: int(v) for k, v in (kv.split("=") for kv in args.override.split(","))})

    def step():
        ops.matmul(A, B, out=C)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    cfg = ops.last_config()

    sampler = ClockSampler(local_rank)
    with sampler:
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        elapsed = time_launches(step, args.steps, stream)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
    if dist is not None:
        t = torch.tensor([elapsed], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = float(t.item())
    status = ops.device_status()
    if status[0] != 0:
        raise SystemExit(f"device-side error {status}: the measurement is void")

    total_flops = 2.0 * M * N * K if name == "sharded" else 2.0 * M * N * K * world
    value = total_flops * args.steps / elapsed / 1e12
    per_launch = elapsed / args.steps
    peaks = roofline.load_measured_peaks()
    sustained = elapsed > 1.0
    roof = roofline.roofline_record(m_rank, N, K, per_launch, peaks, sustained=sustained,
                                    traffic_bytes=NCU_TRAFFIC_BYTES.get(name) if world == 1 else None)

    # ---- cuBLAS through torch.matmul, timed the same way, for context -------------------------
    cublas = None
    if not args.no_cublas:
        Ct = torch.empty_like(C)

        def cublas_step():
            torch.matmul(A, B.t(), out=Ct)
        for _ in range(max(args.warmup, 3)):
            cublas_step()
        torch.cuda.synchronize()
        t_cublas = time_launches(cublas_step, args.steps, stream)
        if dist is not None:
            t = torch.tensor([t_cublas], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_cublas = float(t.item())
        cublas = {"value": total_flops * args.steps / t_cublas / 1e12, "unit": UNIT,
                  "ms_per_step": t_cublas / args.steps * 1e3, "how": "torch.matmul(A, B.t(), out=)"}
        del Ct

    # ---- end to end: host buffers in, host buffer out ----------------------------------------
    e2e = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 10))
        hA = torch.empty((m_rank, K), dtype=torch.bfloat16).pin_memory()
        hB = torch.empty((N, K), dtype=torch.bfloat16).pin_memory()
        hC = torch.empty((m_rank, N), dtype=torch.bfloat16).pin_memory()
        hA.copy_(A)
        hB.copy_(B)
        torch.cuda.synchronize()
        if world == 1:
            def e2e_step():
                ops.matmul_host(hA, hB, hC, device=local_rank)
            h2d = hA.numel() * 2 + hB.numel() * 2
        else:
            # Each rank uploads its block of A; rank 0 uploads B and NCCL broadcasts it.
            def e2e_step():
                A.copy_(hA, non_blocking=True)
                if rank == 0:
                    B.copy_(hB, non_blocking=True)
                dist.broadcast(B, src=0)
                ops.matmul(A, B, out=C)
                hC.copy_(C, non_blocking=True)
                torch.cuda.current_stream().synchronize()
            h2d = hA.numel() * 2 + (hB.numel() * 2 if rank == 0 else 0)
        for _ in range(2):
            e2e_step()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        t_e2e = time_launches(e2e_step, e2e_steps, stream)
        if dist is not None:
            t = torch.tensor([t_e2e], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_e2e = float(t.item())
        e2e = {"value": total_flops * e2e_steps / t_e2e / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(hC.numel() * 2),
               "ms_per_step": t_e2e / e2e_steps * 1e3, "steps": e2e_steps,
               "api": "neogemm_bf16_nt_host (pinned host buffers)" if world == 1 else
                      "pinned H2D of the A block (+B on rank 0) + NCCL broadcast of B + "
                      "neogemm_bf16_nt + pinned D2H of the C block"}
        del hA, hB, hC

    # ---- CPU baseline (rank 0, N = 1 only) -----------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tf, dt, rows = time_cpu_oracle(m_rank, N, K, args.seed, steps=3, warmup=1)
        cpu = {"value": tf, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"first {rows} of {m_rank} rows of A x all {N} rows of B, K={K}; torch "
                         f"CPU fp32 matmul of the bf16 operands (the oracle), mean of 3 runs"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": per_launch * 1e3,
            "higher_is_better": True,
            "scaling": "strong" if name == "sharded" else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": workload_label(name, M, N, K, world),
                "rows_per_gpu": m_rank,
                "l2": "operands + result per launch (%.0f MB) exceed the 126 MB L2; no flush"
                      % ((m_rank * K + N * K + m_rank * N) * 2 / 1e6),
                "kernel": cfg,
            },
            "roofline": roof,
            "e2e": e2e,
            "cpu_baseline": cpu,
            "cublas": cublas,
            "gpu_launches": args.steps,
            "clocks": sampler.record(),
            "per_gpu_tflops": value / world,
            "frac_of_nominal_2250": value / world / 2250.0,
        }
        if bcast_ms is not None:
            line["broadcast_b"] = {"ms": bcast_ms, "bytes": N * K * 2,
                                   "gbs": N * K * 2 / bcast_ms / 1e6, "timed": "separately"}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
