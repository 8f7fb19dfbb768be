"""Algorithmic work of the GEMM path and the peaks it is compared with.

flops = 2*M*N*K; bytes = 2*(M*K + N*K + M*N): each bf16 operand read once and C written once.
Split-K scratch traffic and padded tensor-core rows do not count.  (The reference computes
TFLOPS = 2*M*N*K / t / 1e12 the same way, benchmark.py:57,78,99; cublass/matmul.cu:180-183.)
"""
from __future__ import annotations

import json
from pathlib import Path

NOMINAL_BF16_TFLOPS = 2250.0   # dense
NOMINAL_HBM_GBS = 8000.0
FALLBACK_BF16_TFLOPS = 1590.0  # earlier measurement on the same GPU pool, used if no file
FALLBACK_HBM_GBS = 6650.0


def gemm_flops(M: int, N: int, K: int) -> int:
    return 2 * M * N * K


def gemm_bytes(M: int, N: int, K: int) -> int:
    return 2 * (M * K + N * K + M * N)


def arithmetic_intensity(M: int, N: int, K: int) -> float:
    return gemm_flops(M, N, K) / max(gemm_bytes(M, N, K), 1)


def load_measured_peaks(root: Path | None = None) -> dict:
    """Peaks measured on this GPU pool (MEASURED_PEAKS.json beside the benchmark), else the
    fallback figures; ``source`` says which."""
    root = Path(__file__).resolve().parent.parent if root is None else Path(root)
    f = root / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            d = json.loads(f.read_text())
            return {"bf16_tflops": float(d["bf16_tflops"]),
                    "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
        except (ValueError, KeyError):
            pass
    return {"bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0,
            "hbm_gbs": FALLBACK_HBM_GBS, "source": "fallback"}


def bound_of(M: int, N: int, K: int, peaks: dict) -> str:
    """"tensor" if the shape's arithmetic intensity exceeds the machine balance, else "hbm"."""
    balance = peaks["bf16_tflops"] * 1e12 / (peaks["hbm_gbs"] * 1e9)
    return "tensor" if arithmetic_intensity(M, N, K) >= balance else "hbm"


def roofline_record(M: int, N: int, K: int, seconds_per_launch: float, peaks: dict,
                    sustained: bool = False, traffic_bytes=None) -> dict:
    bound = bound_of(M, N, K, peaks)
    if bound == "tensor":
        achieved = gemm_flops(M, N, K) / seconds_per_launch / 1e12
        peak = peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"]
        unit = "TFLOP/s"
    else:
        achieved = gemm_bytes(M, N, K) / seconds_per_launch / 1e9
        peak = peaks["hbm_gbs"]
        unit = "GB/s"
    return {"bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
            "frac": achieved / peak, "traffic": traffic_bytes,
            "peak_source": peaks["source"] + (" sustained" if (sustained and bound == "tensor") else " burst" if bound == "tensor" else "")}
