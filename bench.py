#!/usr/bin/env python
"""Benchmark of the BF16 GEMM hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One step = one pass of the hot path over one batch of synthetic operands: one GEMM launch per
GPU.  N = 1 runs the headline 8192^3 shape; N > 1 (launched by torchrun, one rank per GPU) runs
the row-sharded 131072 x 8192 x 8192 GEMM: A is split into N contiguous row blocks, B is broadcast
once from rank 0 with NCCL (timed separately), no reduction follows.  Rank 0 prints one JSON line.

`value` is device-timed (CUDA events on the launching stream, max over ranks) with operands
resident in HBM.  `e2e` is the same metric with HOST buffers in and out: through the C ABI's host
entry point at N = 1 and through shard.sharded_matmul_host at N > 1 (uploads, the broadcast of B,
products and downloads overlapped); every host<->device copy is inside the timed region.
`--impl reference` times the CPU restatement of the path (oracle/oracle.py: torch fp32 matmul on
all host cores) - the reference has no CPU implementation and its GPU kernels cannot run on sm_100.

Besides the contract keys the N = 1 line carries, measured after the headline region in the same
process: `cublas` (torch.matmul timed the same way, in alternating blocks with ours),
`sustained` (8192^3 for seconds, ours and cuBLAS in alternating blocks), `configs` (the other
benchmark configurations: decode M = 16/64/128, 4096^3, 512^3, each as CUDA-graph replays beside
cuBLAS, with its roofline fraction) and `sharded_1gpu` (the 8-GPU job on one GPU, the base of
the strong-scaling curve).  The N > 1 line adds `parity` (sampled rows of every rank's result
against the CPU oracle, checksum of the broadcast B), `broadcast_b`, `broadcast_overlap` and the
concurrent PCIe floor of the box inside `e2e`.
"""
from __future__ import annotations

import argparse
import json
import math
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
L2_BYTES = 126e6

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
# The configurations timed besides the headline one in the default N = 1 run: (name, launches per
# CUDA graph).
EXTRA_CONFIGS = (("decode16", 200), ("decode64", 200), ("decode128", 200), ("4096", 40),
                 ("512", 200))


def load_ncu_traffic():
    """DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch of the dominant
    kernel per workload, from profiles/dram_traffic.txt, which also names the commit and capture
    each figure comes from.  Missing file or workload -> None."""
    out = {}
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    try:
        for raw in open(path):
            line = raw.split("#", 1)[0].split()
            if len(line) >= 3:
                out[line[0]] = {"bytes": int(line[1]) + int(line[2]),
                                "captured_at": line[3] if len(line) > 3 else None}
    except (OSError, ValueError):
        pass
    return out


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
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the sustained / other-configurations / 1-GPU sharded legs")
    ap.add_argument("--sustained-seconds", type=float, default=2.0)
    ap.add_argument("--override", default="",
                    help="tuning only: kernel override, e.g. cta_group=2,block_n=256,group_m=8")
    ap.add_argument("--tuning", default="",
                    help="tuning only: knobs of gemm_b200.ops.TUNING_KEYS, e.g. wave_pacing=0")
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

    def __init__(self, device_index: int, period_s: float = 0.001):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period_s = period_s
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
            time.sleep(self.period_s)

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
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_min_mhz": min(self.samples),
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


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
    # Each step is a bounded sample (about 0.15 s on 16 cores); steps and warm-up are the caller's,
    # capped so that the arm ends within a few minutes on any box.
    steps = max(1, min(args.steps, 200))
    warmup = max(0, min(args.warmup, 50))
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


def max_over_ranks(dist, seconds, device):
    if dist is None:
        return seconds
    t = torch.tensor([seconds], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def l2_note(bytes_per_set, sets):
    if bytes_per_set > L2_BYTES:
        return "operands + result per launch (%.0f MB) exceed the 126 MB L2; no flush" % (
            bytes_per_set / 1e6)
    if bytes_per_set * (sets - 1) > L2_BYTES:
        return ("%.0f MB per launch fit the 126 MB L2: launches rotate through %d operand sets "
                "(%.0f MB), so every launch starts L2-cold" % (bytes_per_set / 1e6, sets,
                                                             bytes_per_set * sets / 1e6))
    return ("%.1f MB per launch fit the 126 MB L2: timed L2-warm (back-to-back launches on %d "
            "operand set(s))" % (bytes_per_set / 1e6, sets))


def time_graph(calls, replays):
    """Captures `calls` (a list of launch closures) into one CUDA graph and returns the mean
    device time of one call over `replays` replays (after one untimed replay)."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in calls[:4]:
            f()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for f in calls:
            f()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    e1.synchronize()
    return e0.elapsed_time(e1) / 1e3 / (replays * len(calls))


def run_extra_config(name, launches, seed, device, peaks, ops, roofline, traffic):
    """One of the other benchmark configurations on one GPU: ours and cuBLAS as CUDA-graph
    replays of `launches` back-to-back launches rotating through operand sets."""
    M, N, K = WORKLOADS[name]
    per_set = roofline.gemm_bytes(M, N, K)
    sets = 2 if per_set > L2_BYTES else max(1, min(4, math.ceil(2 * L2_BYTES / per_set)))
    As = [device_operand(M, K, seed + 100 + i, device) for i in range(sets)]
    Bs = [device_operand(N, K, seed + 200 + i, device) for i in range(sets)]
    Cs = [torch.empty((M, N), dtype=torch.bfloat16, device=device) for _ in range(sets)]
    ours_calls = [(lambda i=i: ops.matmul(As[i % sets], Bs[i % sets], out=Cs[i % sets]))
                  for i in range(launches)]
    cublas_calls = [(lambda i=i: torch.matmul(As[i % sets], Bs[i % sets].t(), out=Cs[i % sets]))
                    for i in range(launches)]
    ours_calls[0]()
    cfg = ops.last_config()
    cfg["store_path"] = ops.last_store_path()   # 1 / 2: a tall tile left as one TMA box
    replays = 5
    t_ours = time_graph(ours_calls, replays)
    t_cublas = time_graph(cublas_calls, replays)
    t_ours2 = time_graph(ours_calls, replays)
    t_ours = min(t_ours, t_ours2)
    status = ops.device_status()
    if status[0] != 0:
        raise SystemExit(f"device-side error {status} in configuration {name}")
    roof = roofline.roofline_record(M, N, K, t_ours, peaks, sustained=False,
                                    traffic_bytes=(traffic.get(name) or {}).get("bytes"))
    rec = {
        "name": name, "workload": workload_label(name, M, N, K, 1), "us": t_ours * 1e6,
        "cublas_us": t_cublas * 1e6, "vs_cublas": t_cublas / t_ours,
        "launches": launches * replays, "timed": f"CUDA-graph replays of {launches} launches, "
                                                 f"{replays} replays, best of two runs for ours",
        "l2": l2_note(per_set, sets), "kernel": cfg, "roofline": roof,
        "tflops": 2.0 * M * N * K / t_ours / 1e12,
    }
    if roof["bound"] == "hbm":
        rec["frac_of_nominal_8000_gbs"] = roof["achieved"] / roofline.NOMINAL_HBM_GBS
    del As, Bs, Cs
    return rec


def run_sustained(step_ours, step_cublas, flops_per_step, seconds, stream, local_rank):
    """Seconds of continuous load: blocks of launches alternate between ours and cuBLAS, so both
    see the same power and thermal state; each side's figure is its own launches over its own
    accumulated device time."""
    block = 100
    acc = {"ours": 0.0, "cublas": 0.0}
    n = {"ours": 0, "cublas": 0}
    sampler = ClockSampler(local_rank, period_s=0.01)
    with sampler:
        while min(acc.values()) < seconds and sum(acc.values()) < 6 * seconds:
            for key, fn in (("ours", step_ours), ("cublas", step_cublas)):
                acc[key] += time_launches(fn, block, stream)
                n[key] += block
    out = {k: {"value": flops_per_step * n[k] / acc[k] / 1e12, "unit": UNIT,
               "ms_per_step": acc[k] / n[k] * 1e3, "launches": n[k], "seconds": acc[k]}
           for k in acc}
    out["ratio_to_cublas"] = out["ours"]["value"] / out["cublas"]["value"]
    out["protocol"] = (f"alternating blocks of {block} launches, ours then cuBLAS, until each "
                       f"side has {seconds:g} s of device time")
    out["clocks"] = sampler.record()
    return out


def pcie_floor(h2d_pairs, d2h_pairs, device, dist, reps=3):
    """Time of the step's host<->device bytes alone: every upload on one stream, every download
    on another, both directions at once, all ranks at the same time (max over ranks)."""
    cur = torch.cuda.current_stream(device)
    s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)

    def once():
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            for dst, src in h2d_pairs:
                dst.copy_(src, non_blocking=True)
        with torch.cuda.stream(s_out):
            for dst, src in d2h_pairs:
                dst.copy_(src, non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
    once()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
    t = time_launches(once, reps, cur) / reps
    return max_over_ranks(dist, t, device)


def b_checksum(B):
    v = B.view(torch.int16).to(torch.int64)
    rows = torch.arange(1, B.shape[0] + 1, device=B.device, dtype=torch.int64).unsqueeze(1)
    return torch.stack([v.sum(), (v * (rows % 65521)).sum()])


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
    r0 = 0
    if name == "sharded":
        from gemm_b200.shard import row_partition
        r0, r1 = row_partition(M, world, rank)
        m_rank = r1 - r0
    else:
        m_rank = M
    stream = torch.cuda.current_stream(device)
    traffic = load_ncu_traffic()

    # ---- operands resident in HBM -----------------------------------------------------------
    A = device_operand(m_rank, K, args.seed + 17 * (rank + 1), device)
    # Multi-GPU runs check sampled rows of every rank's result after the timed regions: three
    # 256-row slices of the A block come from the CPU-seeded generator (any rank can regenerate
    # any slice from (seed, global row) alone) and are written over the device-generated rows.
    sampled = []
    if world > 1:
        from gemm_b200.inputs import make_row_block
        for s0 in sorted({0, (m_rank // 2) // 256 * 256, max(0, m_rank - 256)}):
            rows = min(256, m_rank - s0)
            A[s0:s0 + rows] = make_row_block((r0 + s0) // 256, rows, K, args.seed).to(device)
            sampled.append((s0, rows))
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
        bcast_ms = max_over_ranks(dist, e0.elapsed_time(e1) / 1e3, device) * 1e3
    else:
        B = device_operand(N, K, args.seed, device)
    C = torch.empty((m_rank, N), dtype=torch.bfloat16, device=device)

    if args.override:
        ops.set_override(**{k: int(v) for k, v in (kv.split("=") for kv in args.override.split(","))})
    if args.tuning:
        for kv in args.tuning.split(","):
            k, v = kv.split("=")
            ops.set_tuning(k, int(v))

    def step():
        ops.matmul(A, B, out=C)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    cfg = ops.last_config()
    cfg["store_path"] = ops.last_store_path()

    sampler = ClockSampler(local_rank)
    with sampler:
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        elapsed = time_launches(step, args.steps, stream)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
    elapsed = max_over_ranks(dist, elapsed, device)
    status = ops.device_status()
    if status[0] != 0:
        raise SystemExit(f"device-side error {status}: the measurement is void")

    flops_per_step = 2.0 * M * N * K if name == "sharded" else 2.0 * M * N * K * world
    value = flops_per_step * args.steps / elapsed / 1e12
    per_launch = elapsed / args.steps
    peaks = roofline.load_measured_peaks()
    sustained_regime = elapsed > 1.0
    tr = traffic.get(name) if world == 1 else None
    roof = roofline.roofline_record(m_rank, N, K, per_launch, peaks, sustained=sustained_regime,
                                    traffic_bytes=tr["bytes"] if tr else None)
    if tr:
        roof["traffic_source"] = f"profiles/dram_traffic.txt ({tr['captured_at']})"

    # ---- cuBLAS through torch.matmul, timed the same way, then ours and cuBLAS once more -------
    cublas = None
    Ct = None
    if not args.no_cublas:
        Ct = torch.empty_like(C)

        def cublas_step():
            torch.matmul(A, B.t(), out=Ct)
        for _ in range(warmup):
            cublas_step()
        torch.cuda.synchronize()
        t_cublas = max_over_ranks(dist, time_launches(cublas_step, args.steps, stream), device)
        t_ours_2 = max_over_ranks(dist, time_launches(step, args.steps, stream), device)
        t_cublas_2 = max_over_ranks(dist, time_launches(cublas_step, args.steps, stream), device)
        to_tf = lambda t: flops_per_step * args.steps / t / 1e12  # noqa: E731
        cublas = {"value": to_tf(t_cublas), "unit": UNIT,
                  "ms_per_step": t_cublas / args.steps * 1e3, "how": "torch.matmul(A, B.t(), out=)",
                  "order": "ours (the line's value), cuBLAS (this value), ours again, cuBLAS again; "
                           f"{args.steps} launches each, back to back",
                  "ours_again": to_tf(t_ours_2), "cublas_again": to_tf(t_cublas_2)}

    # ---- end to end: host buffers in, host buffer out ----------------------------------------
    e2e = None
    e2e_rows_ok = None
    if not args.no_e2e:
        e2e_steps = max(3, min(args.steps, 10))
        hA = torch.empty((m_rank, K), dtype=torch.bfloat16).pin_memory()
        hB = torch.empty((N, K), dtype=torch.bfloat16).pin_memory() if (rank == 0) else None
        hC = torch.empty((m_rank, N), dtype=torch.bfloat16).pin_memory()
        hA.copy_(A)
        if hB is not None:
            hB.copy_(B)
        torch.cuda.synchronize()
        if world == 1:
            def e2e_step():
                ops.matmul_host(hA, hB, hC, device=local_rank)
            h2d = hA.numel() * 2 + hB.numel() * 2
            floor_h2d = [(A, hA), (B, hB)]
            api = "neogemm_bf16_nt_host (pinned host buffers)"
        else:
            from gemm_b200.shard import ShardedHostPipeline
            pipe = ShardedHostPipeline(m_rank, N, K, device)

            def e2e_step():
                pipe.run(hA, hB, hC)
            h2d = pipe.h2d_bytes(rank)
            floor_h2d = [(A, hA)] + ([(B, hB)] if rank == 0 else [])
            api = ("shard.sharded_matmul_host: pinned H2D of the A block in row chunks (+ B on "
                   "rank 0, chunk by chunk into the NCCL broadcast), one neogemm_bf16_nt per "
                   "landed chunk, pinned D2H of finished rows, all overlapped")
        for _ in range(2):
            e2e_step()
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()
        t_e2e = max_over_ranks(dist, time_launches(e2e_step, e2e_steps, stream), device)
        if world > 1:
            # keep the last step's host result for the parity leg
            e2e_rows = [(s0, hC[s0:s0 + rows].clone()) for s0, rows in sampled]
        floor_s = pcie_floor(floor_h2d, [(hC, C)], device, dist)
        e2e = {"value": flops_per_step * e2e_steps / t_e2e / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(hC.numel() * 2),
               "ms_per_step": t_e2e / e2e_steps * 1e3, "steps": e2e_steps, "api": api,
               "pcie_floor_ms": floor_s * 1e3,
               "pcie_floor_how": "the step's uploads on one stream and its download on another, "
                                 "both at once, all ranks at once, pinned buffers, max over ranks",
               "x_pcie_floor": t_e2e / e2e_steps / floor_s}
        if world > 1:
            del pipe
        del hA, hB, hC

    # ---- N > 1: the broadcast of B hidden under compute, or not --------------------------------
    overlap = None
    if world > 1:
        from gemm_b200.shard import sharded_matmul_overlapped

        def serial_step():
            dist.broadcast(B, src=0)
            ops.matmul(A, B, out=C)

        def overlapped_step(chunks):
            return lambda: sharded_matmul_overlapped(A, B if rank == 0 else None, N, K,
                                                     chunks=chunks, out=C, B_buffer=B)
        times = {}
        for key, fn in (("serial", serial_step), ("overlapped2", overlapped_step(2)),
                        ("overlapped4", overlapped_step(4))):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            times[key] = max_over_ranks(dist, time_launches(fn, 5, stream), device) / 5
        overlap = {"broadcast_then_gemm_ms": times["serial"] * 1e3,
                   "broadcast_under_gemm_2_chunks_ms": times["overlapped2"] * 1e3,
                   "broadcast_under_gemm_4_chunks_ms": times["overlapped4"] * 1e3,
                   "gemm_alone_ms": per_launch * 1e3, "broadcast_alone_ms": bcast_ms,
                   "how": "5 steps each, CUDA events, max over ranks; overlapped = "
                          "shard.sharded_matmul_overlapped (B in row chunks on a side stream, "
                          "one product per landed chunk, buffers kept across calls)"}

    # ---- N > 1: parity of sampled rows and of the broadcast, untimed ---------------------------
    parity = None
    if world > 1:
        from gemm_b200.inputs import make_row_block
        from oracle import oracle
        torch.set_num_threads(max(1, min(8, (os.cpu_count() or 8) // world)))
        C.fill_(float("nan"))
        step()
        torch.cuda.synchronize()
        B_cpu = B.cpu()
        rows_checked, max_ulp, bit_equal, ok = 0, 0, 1.0, True
        e2e_rows_ok = True if not args.no_e2e else None
        for i, (s0, rows) in enumerate(sampled):
            a_rows = make_row_block((r0 + s0) // 256, rows, K, args.seed)
            ref = oracle.gemm_fp32(a_rows, B_cpu)
            try:
                s = oracle.assert_parity(C[s0:s0 + rows], ref, f"rank {rank} rows {r0 + s0}..")
                max_ulp = max(max_ulp, s["max_ulp"])
                bit_equal = min(bit_equal, s["bit_equal_frac"])
            except AssertionError as e:
                ok = False
                print(f"PARITY FAILURE: {e}", file=sys.stderr, flush=True)
            if e2e_rows_ok is not None:
                try:
                    oracle.assert_parity(e2e_rows[i][1], ref, f"rank {rank} e2e rows {r0 + s0}..")
                except AssertionError as e:
                    e2e_rows_ok = False
                    print(f"PARITY FAILURE (e2e): {e}", file=sys.stderr, flush=True)
            rows_checked += rows
        sums = [torch.empty(2, dtype=torch.int64, device=device) for _ in range(world)]
        dist.all_gather(sums, b_checksum(B))
        stats = torch.tensor([rows_checked, max_ulp, int(bit_equal * 1e9), int(ok),
                              int(e2e_rows_ok is not False)], device=device, dtype=torch.int64)
        gathered = [torch.empty_like(stats) for _ in range(world)]
        dist.all_gather(gathered, stats)
        g = torch.stack(gathered).cpu()
        parity = {"rows_checked": int(g[:, 0].sum()), "ranks": world,
                  "max_ulp": int(g[:, 1].max()), "bit_equal_frac": float(g[:, 2].min()) / 1e9,
                  "all_gates_ok": bool(g[:, 3].min() == 1),
                  "b_checksum_ok": all(bool(torch.equal(s, sums[0])) for s in sums),
                  "e2e_rows_ok": (bool(g[:, 4].min() == 1) if not args.no_e2e else None),
                  "how": "three 256-row slices of every rank's A block are CPU-seeded; their rows "
                         "of C (device-resident step, and the last e2e step's host buffer) are "
                         "checked with the CPU oracle's gates (allclose 1e-2, rel. Frobenius "
                         "<= 3e-3, >= 98 % bit-equal, <= 1 ulp); every rank's B is checksummed "
                         "against rank 0's"}
        if not (parity["all_gates_ok"] and parity["b_checksum_ok"]) or parity["e2e_rows_ok"] is False:
            if rank == 0:
                print(json.dumps({"parity": parity}), file=sys.stderr, flush=True)
            raise SystemExit("parity failure in the sharded run: the measurement is void")

    # ---- CPU baseline (rank 0, N = 1 only) -----------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tf, dt, rows = time_cpu_oracle(m_rank, N, K, args.seed, steps=3, warmup=1)
        cpu = {"value": tf, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
               "sample": f"first {rows} of {m_rank} rows of A x all {N} rows of B, K={K}; torch "
                         f"CPU fp32 matmul of the bf16 operands (the oracle), mean of 3 runs"}

    # ---- N = 1 default run: sustained load, the other configurations, the 1-GPU sharded base ----
    sustained = configs = sharded_1gpu = None
    extras = world == 1 and name == "8192" and not args.no_extras and not args.override \
        and not args.tuning
    if extras:
        if Ct is None:
            Ct = torch.empty_like(C)
        sustained = run_sustained(step, lambda: torch.matmul(A, B.t(), out=Ct), flops_per_step,
                                  args.sustained_seconds, stream, local_rank)
        sustained["roofline_frac_of_sustained_peak"] = (
            sustained["ours"]["value"] / peaks["bf16_tflops_sustained"])
        del A, B, C, Ct
        torch.cuda.empty_cache()
        configs = [run_extra_config(n, launches, args.seed, device, peaks, ops, roofline, traffic)
                   for n, launches in EXTRA_CONFIGS]
        torch.cuda.empty_cache()
        Ms, Ns, Ks = WORKLOADS["sharded"]
        A = device_operand(Ms, Ks, args.seed + 17, device)
        B = device_operand(Ns, Ks, args.seed, device)
        C = torch.empty((Ms, Ns), dtype=torch.bfloat16, device=device)
        for _ in range(3):
            step()
        big_cfg = ops.last_config()
        for _ in range(3):
            torch.matmul(A, B.t(), out=C)
        torch.cuda.synchronize()
        n_big = 10
        t_o = time_launches(step, n_big, stream)
        t_c = time_launches(lambda: torch.matmul(A, B.t(), out=C), n_big, stream)
        t_o2 = time_launches(step, n_big, stream)
        t_c2 = time_launches(lambda: torch.matmul(A, B.t(), out=C), n_big, stream)
        fl = 2.0 * Ms * Ns * Ks * n_big / 1e12
        sharded_1gpu = {"workload": workload_label("sharded", Ms, Ns, Ks, 1),
                        "value": fl / min(t_o, t_o2), "unit": UNIT,
                        "ms_per_step": min(t_o, t_o2) / n_big * 1e3,
                        "cublas": fl / min(t_c, t_c2), "kernel": big_cfg,
                        "how": f"{n_big} launches per block, blocks ours / cuBLAS / ours / cuBLAS, "
                               "best block of each"}
        status = ops.device_status()
        if status[0] != 0:
            raise SystemExit(f"device-side error {status} in the extra legs")

    if rank == 0:
        per_set = (m_rank * K + N * K + m_rank * N) * 2
        launches = args.steps
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warmup, "ms_per_step": per_launch * 1e3,
            "higher_is_better": True,
            "scaling": "strong" if name == "sharded" else "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": workload_label(name, M, N, K, world),
                "rows_per_gpu": m_rank,
                "l2": l2_note(per_set, 1),
                "kernel": cfg,
            },
            "roofline": roof,
            "e2e": e2e,
            "cpu_baseline": cpu,
            "cublas": cublas,
            "gpu_launches": launches,
            "clocks": sampler.record(),
            "per_gpu_tflops": value / world,
            "frac_of_nominal_2250": value / world / 2250.0,
        }
        if bcast_ms is not None:
            line["broadcast_b"] = {"ms": bcast_ms, "bytes": N * K * 2,
                                   "gbs": N * K * 2 / bcast_ms / 1e6, "timed": "separately"}
        if overlap is not None:
            line["broadcast_overlap"] = overlap
        if parity is not None:
            line["parity"] = parity
        if sustained is not None:
            line["sustained"] = sustained
        if configs is not None:
            line["configs"] = configs
        if sharded_1gpu is not None:
            line["sharded_1gpu"] = sharded_1gpu
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
