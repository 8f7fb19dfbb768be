"""GPU: second opinions on the kernel's results, beyond the CPU oracle.

1. Bit-level comparison with cuBLAS (torch.matmul on the same device), the comparison the
   reference's own driver performs (benchmark.py:18,33-53) and its harness is built around
   (cublass/matmul.cu:130-149): at every benchmark configuration and at ragged shapes the two
   bf16 results may differ by at most one ulp, and the bit-equal fraction is reported.
2. The per-GPU shapes of the row-sharded benchmark job (131072 x 8192 x 8192 over 8 and 2 GPUs:
   16384 and 65536 rows): full and sampled-block parity against the CPU oracle with the plan the
   launcher picks on its own (two-half pair tile on all 148 SMs, raster groups of 16 tile rows,
   wave pacing from 8 waves on), and bit-identical results over repeated launches.
3. The stand-alone C++ verify/timing tool (cublass/matmul.cu, counterpart of the reference's
   cublass/matmul.cu:45-51,61-75,170-183) is built with make and run on a ragged shape.
"""
import os
import shutil
import subprocess

import pytest
import torch

from gemm_b200 import ops
from gemm_b200.inputs import make_problem
from oracle import oracle
from tests.util import gpu_bits_compare

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def device_operand(rows, K, seed):
    """Seeded N(0,1)/sqrt(K) operand generated on the device (the tall shapes would take the CPU
    generator tens of seconds); the CPU oracle is fed copies of the same bits."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = torch.empty((rows, K), dtype=torch.bfloat16, device="cuda")
    for r in range(0, rows, 8192):
        n = min(8192, rows - r)
        out[r:r + n] = (torch.randn(n, K, generator=g, device="cuda") / (K ** 0.5)).to(torch.bfloat16)
    return out


def cublas_product(dA, dB):
    """cuBLAS through torch, with fp32 accumulation end to end (no reduced-precision split-K)."""
    flag = torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    try:
        return torch.matmul(dA, dB.t())
    finally:
        torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = flag


def check_against_cublas(dA, dB, what, col_major=False):
    M, N = dA.shape[0], dB.shape[0]
    if col_major:
        C = torch.full((N, M), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.neoGemmV1(dA, dB, C)
        ours = C.t()
    else:
        ours = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        ops.matmul(dA, dB, out=ours)
    cfg = ops.last_config()
    theirs = cublas_product(dA, dB)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    s = gpu_bits_compare(ours, theirs)
    print(f"cuBLAS cross-check {what}: bit-equal {s['bit_equal_frac']:.6f} of {s['elements']}, "
          f"max {s['max_ulp']} ulp, cfg={cfg}")
    assert s["finite"], (what, s)
    assert s["max_ulp"] <= 1 and s["near_zero_ok"], (what, s, cfg)
    assert s["bit_equal_frac"] >= 0.98, (what, s, cfg)
    return s


@pytest.mark.parametrize("shape", [(512, 512, 512), (4096, 4096, 4096), (8192, 8192, 8192),
                                   (16, 28672, 8192), (64, 28672, 8192), (128, 28672, 8192),
                                   (16384, 8192, 8192),            # one rank's share of 8 GPUs
                                   (1000, 1001, 520), (300, 776, 1352), (33, 20008, 1536)])
def test_bits_against_cublas(shape):
    M, N, K = shape
    if M * K > (1 << 26):
        dA, dB = device_operand(M, K, 21), device_operand(N, K, 22)
    else:
        A, B = make_problem(M, N, K, seed=1234)
        dA, dB = A.cuda(), B.cuda()
    check_against_cublas(dA, dB, f"{M}x{N}x{K}")
    if M <= 4096:
        check_against_cublas(dA, dB, f"{M}x{N}x{K} column-major", col_major=True)


def _expect_wide_pair_plan(cfg, tiles):
    assert (cfg["cta_group"], cfg["block_n"], cfg["ctas"], cfg["stream_k"]) == (2, 512, 148, 0), cfg
    assert cfg["tiles"] == tiles and cfg["group_m"] == 16, cfg


def test_sharded_job_share_of_eight_gpus_in_full():
    # 16384 x 8192 x 8192: 1024 two-half tiles on 74 CTA pairs (13.8 waves), wave pacing on.
    M, N, K = 16384, 8192, 8192
    dA, dB = device_operand(M, K, 31), device_operand(N, K, 32)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.matmul(dA, dB, out=out)
    _expect_wide_pair_plan(ops.last_config(), 1024)
    first = out.clone()
    for _ in range(4):
        ops.matmul(dA, dB, out=out)
        assert torch.equal(first.view(torch.int16), out.view(torch.int16)), "launches differ"
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    B = dB.cpu()
    worst = {"bit_equal_frac": 1.0, "max_ulp": 0}
    for r0 in range(0, M, 2048):
        ref = oracle.gemm_fp32(dA[r0:r0 + 2048].cpu(), B)
        s = oracle.assert_parity(first[r0:r0 + 2048], ref, f"16384-row share, rows {r0}..")
        worst["bit_equal_frac"] = min(worst["bit_equal_frac"], s["bit_equal_frac"])
        worst["max_ulp"] = max(worst["max_ulp"], s["max_ulp"])
    print("16384 x 8192 x 8192 in full:", worst)


def test_sharded_job_share_of_two_gpus_on_sampled_blocks():
    # 65536 x 8192 x 8192: 4096 tiles, 55 waves.  256-row blocks against the oracle: the first
    # and last rows, blocks either side of raster-group boundaries (4096 rows) and odd ones.
    M, N, K = 65536, 8192, 8192
    dA, dB = device_operand(M, K, 41), device_operand(N, K, 42)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.matmul(dA, dB, out=out)
    _expect_wide_pair_plan(ops.last_config(), 4096)
    first = out.clone()
    for _ in range(4):
        ops.matmul(dA, dB, out=out)
        assert torch.equal(first.view(torch.int16), out.view(torch.int16)), "launches differ"
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 0
    assert bool(torch.isfinite(first).all()), "unwritten (NaN-poisoned) elements"
    B = dB.cpu()
    for r0 in (0, 3840, 4096, 20224, 32768 - 256, 32768, 49152 + 768, M - 256):
        ref = oracle.gemm_fp32(dA[r0:r0 + 256].cpu(), B)
        oracle.assert_parity(first[r0:r0 + 256], ref, f"65536-row share, rows {r0}..{r0 + 256}")
    # and every element against cuBLAS on the device
    s = gpu_bits_compare(first, cublas_product(dA, dB))
    print("65536 x 8192 x 8192 against cuBLAS:", s)
    assert s["max_ulp"] <= 1 and s["near_zero_ok"] and s["bit_equal_frac"] >= 0.98, s


@pytest.mark.timeout(600)
def test_cpp_verify_and_timing_tool_builds_and_agrees():
    if shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"):
        pytest.skip("no nvcc on this machine: the C++ tool cannot be built")
    env = dict(os.environ)
    env["PATH"] = env.get("PATH", "") + os.pathsep + "/usr/local/cuda/bin"
    made = subprocess.run(["make", "-C", os.path.join(ROOT, "cublass"), "matmul"],
                          capture_output=True, text=True, env=env, timeout=500)
    assert made.returncode == 0, made.stdout[-2000:] + made.stderr[-2000:]
    exe = os.path.join(ROOT, "cublass", "out", "matmul")
    for args in (["520", "776", "1352"], ["16", "3584", "2048"]):
        run = subprocess.run([exe, *args, "--iters", "2", "--timers"], capture_output=True,
                             text=True, env=env, timeout=120)
        assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
        assert ", 0 outside rtol" in run.stdout, run.stdout
        assert "Divergence" not in run.stdout
        assert "phase timers over" in run.stdout


@pytest.mark.timeout(300)
def test_reference_style_driver_script_runs_and_agrees():
    """benchmark.py, the counterpart of the reference's driver (benchmark.py:10-25,33-53,63-100):
    builds operands, calls neoGEMM.neoGemmV1 through the torch extension, compares with torch's
    matmul on the GPU and times both.  Run as the reference's users run it."""
    pytest.importorskip("neoGEMM")
    import sys
    for args in (["--iters", "5"], ["--m", "520", "--n", "776", "--k", "264", "--scaled", "--iters", "2"]):
        run = subprocess.run([sys.executable, os.path.join(ROOT, "benchmark.py"), *args],
                             capture_output=True, text=True, timeout=240, cwd=ROOT)
        assert run.returncode == 0, run.stdout[-2000:] + run.stderr[-2000:]
        assert "tolerance 1e-02: PASS" in run.stdout, run.stdout
        assert "neoGEMM:" in run.stdout and "TFLOPS" in run.stdout
