"""Shared helpers for the GPU parity tests (the checker is the CPU oracle)."""
import torch

from gemm_b200 import ops
from gemm_b200.inputs import make_problem
from oracle import oracle


def run_case(M, N, K, col_major=False, seed=1234, override=None, scale_by_k=True, what=None,
             expect=None, tuning=None, **gates):
    """One parity case through the C ABI: seeded operands -> GPU kernel -> compare with oracle.
    The output is poisoned with NaN first so unwritten elements cannot pass."""
    A, B = make_problem(M, N, K, seed=seed, scale_by_k=scale_by_k)
    dA, dB = A.cuda(), B.cuda()
    try:
        if override:
            ops.set_override(**override)
        for key, value in (tuning or {}).items():
            ops.set_tuning(key, value)
        if col_major:
            C = torch.full((N, M), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.neoGemmV1(dA, dB, C)
            out = C.t()
        else:
            C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.matmul(dA, dB, out=C)
            out = C
        cfg = ops.last_config()
    finally:
        if override:
            ops.set_override()
        for key in (tuning or {}):
            ops.set_tuning(key, -1)
    torch.cuda.synchronize()
    status = ops.device_status()
    assert status[0] == 0, f"device reported {status} for {M}x{N}x{K} cfg={cfg}"
    if expect:
        for k, v in expect.items():
            assert cfg[k] == v, f"expected {k}={v}, launcher chose {cfg}"
    ref = oracle.gemm_fp32(A, B)
    label = what or f"{M}x{N}x{K} col_major={col_major} cfg={cfg}"
    stats = oracle.assert_parity(out, ref, label, **gates)
    return stats, cfg


def gpu_bits_compare(out: torch.Tensor, other: torch.Tensor) -> dict:
    """Bit-level comparison of two bf16 matrices ON THE GPU (both results of a GPU kernel, e.g.
    ours and cuBLAS'): fraction of bit-equal elements and the largest distance in bf16 ulps.
    Elements within 2^-6 of the RMS magnitude of zero are judged by absolute error, as in
    oracle.compare (an ulp next to zero means nothing)."""
    assert out.is_cuda and other.is_cuda and out.dtype == other.dtype == torch.bfloat16
    assert out.shape == other.shape
    def key(t):
        b = t.contiguous().view(torch.int16).to(torch.int32) & 0xFFFF
        return torch.where(b >= 0x8000, 0x8000 - b, b)
    ulp = (key(out) - key(other)).abs()
    r = other.float()
    rms = float(r.double().pow(2).mean().sqrt()) if r.numel() else 0.0
    small = r.abs() < rms * 2.0 ** -6
    big_ulp = ulp[~small]
    small_err = (out.float() - r).abs()[small]
    return {
        "finite": bool(torch.isfinite(out).all()) and bool(torch.isfinite(other).all()),
        "bit_equal_frac": float((ulp == 0).float().mean()) if ulp.numel() else 1.0,
        "max_ulp": int(big_ulp.max()) if big_ulp.numel() else 0,
        "near_zero_ok": bool((small_err <= rms * 2.0 ** -6 * 2.0 ** -7).all())
        if small_err.numel() else True,
        "elements": int(ulp.numel()),
    }
