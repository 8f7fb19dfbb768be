"""Python face of the operator, calling the C ABI through ctypes.

Mirrors the reference's binding (module ``neoGEMM``, function ``neoGemmV1(A, B, C)``,
nemgemmV03.cu:396-398; legacy ``neogemm(A, B, C)``, neogemmV02.cu:304-306) with the same argument
names and in-place, column-major result (neogemmV02.cu:236,242; benchmark.py:25), and adds the
row-major forms a caller usually wants.  Unlike the reference it validates its arguments
(the reference takes raw ``data_ptr``s unchecked, nemgemmV03.cu:349-351) and launches on torch's
current stream rather than the legacy default stream (nemgemmV03.cu:383).

torch is used here for device memory and streams only.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib
from ._lib import NeoGemmError, check, lib


def _require_cuda_bf16_matrix(name: str, t: torch.Tensor) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise ValueError(f"{name} must live on a CUDA device (there is no CPU path)")
    if t.dtype != torch.bfloat16:
        raise TypeError(f"{name} must be bfloat16, got {t.dtype}")
    if t.dim() != 2:
        raise ValueError(f"{name} must be 2-D, got shape {tuple(t.shape)}")


def _row_pitch(name: str, t: torch.Tensor) -> int:
    """Leading dimension in elements of a matrix whose rows are contiguous."""
    if t.size(1) > 1 and t.stride(1) != 1:
        raise ValueError(f"{name} must have unit stride along its last dimension")
    if t.size(0) > 1:
        return int(t.stride(0))
    return max(int(t.size(1)), 1)


def _stream_ptr(device: torch.device) -> int:
    return int(torch.cuda.current_stream(device).cuda_stream)


def _launch(A, B, C, M, N, K, lda, ldb, ldc, col_major, workspace: Optional[torch.Tensor]):
    ws_ptr, ws_bytes = None, 0
    if workspace is not None:
        ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel() * workspace.element_size()
    with torch.cuda.device(A.device):
        rc = lib.neogemm_bf16_nt(A.data_ptr(), B.data_ptr(), C.data_ptr(), M, N, K, lda, ldb, ldc,
                                 1 if col_major else 0, ws_ptr, ws_bytes, _stream_ptr(A.device))
    check(rc)


def _check_operands(A: torch.Tensor, B: torch.Tensor):
    _require_cuda_bf16_matrix("A", A)
    _require_cuda_bf16_matrix("B", B)
    if A.device != B.device:
        raise ValueError("A and B must be on the same device")
    M, K = int(A.size(0)), int(A.size(1))
    N = int(B.size(0))
    if int(B.size(1)) != K:
        raise ValueError(f"A is [M,K]=[{M},{K}] but B is [N,K]=[{N},{int(B.size(1))}]: K differs")
    return M, N, K


def neoGemmV1(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> None:
    """C <- A * B^T, written COLUMN-major into C's storage (element (i,j) at offset j*M + i),
    exactly as the reference does; ``C.t()`` of an [M,N]-shaped contiguous C then views the
    product (benchmark.py:24-25).  A is [M,K], B is [N,K], both bf16 with contiguous rows;
    C is a contiguous bf16 tensor with M*N elements.  Returns None."""
    M, N, K = _check_operands(A, B)
    if not isinstance(C, torch.Tensor) or not C.is_cuda or C.dtype != torch.bfloat16:
        raise TypeError("C must be a CUDA bfloat16 tensor")
    if C.device != A.device:
        raise ValueError("C must be on the same device as A and B")
    if C.numel() != M * N or not C.is_contiguous():
        raise ValueError(f"C must be contiguous with M*N = {M * N} elements")
    _launch(A, B, C, M, N, K, _row_pitch("A", A), _row_pitch("B", B), max(M, 1), True, None)


def neogemm(A: torch.Tensor, B: torch.Tensor, C: torch.Tensor) -> None:
    """Legacy name of :func:`neoGemmV1` (module ``neogemm``, neogemmV02.cu:304-306)."""
    neoGemmV1(A, B, C)


def matmul(A: torch.Tensor, B: torch.Tensor, out: Optional[torch.Tensor] = None,
           workspace: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row-major product: returns C[M,N] = A[M,K] * B[N,K]^T in bf16 (fp32 accumulation).
    ``out`` may be any bf16 [M,N] tensor with contiguous rows (its row stride is honoured)."""
    M, N, K = _check_operands(A, B)
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    else:
        _require_cuda_bf16_matrix("out", out)
        if tuple(out.shape) != (M, N) or out.device != A.device:
            raise ValueError(f"out must be [{M},{N}] on {A.device}")
    _launch(A, B, out, M, N, K, _row_pitch("A", A), _row_pitch("B", B), _row_pitch("out", out),
            False, workspace)
    return out


ACTIVATIONS = {"none": 0, "relu": 1, "gelu_tanh": 2}


def matmul_fused(A: torch.Tensor, B: torch.Tensor, out: Optional[torch.Tensor] = None,
                 alpha: float = 1.0, beta: float = 0.0, bias: Optional[torch.Tensor] = None,
                 activation: str = "none", col_major: bool = False,
                 out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """out = act(alpha * A @ B^T + beta * out + bias), in fp32 on the accumulator, rounded once.
    ``bias`` is a bf16 vector of length N; ``out`` is required when beta != 0.  With
    ``col_major`` the result is stored as neoGemmV1 stores it (``out`` is then [N,M]).
    ``out_dtype`` (or the dtype of ``out``) may be torch.float32: the result is then stored
    unrounded, and the beta term is read as fp32."""
    M, N, K = _check_operands(A, B)
    shape = (N, M) if col_major else (M, N)
    if out_dtype is None:
        out_dtype = out.dtype if out is not None else torch.bfloat16
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("out_dtype must be torch.bfloat16 or torch.float32")
    if out is None:
        if beta != 0.0:
            raise ValueError("beta != 0 needs the tensor to accumulate into (out=)")
        out = torch.empty(shape, dtype=out_dtype, device=A.device)
    else:
        if not out.is_cuda or out.dim() != 2 or out.dtype != out_dtype:
            raise TypeError(f"out must be a 2-D CUDA tensor of dtype {out_dtype}")
        if tuple(out.shape) != shape or out.device != A.device:
            raise ValueError(f"out must be {list(shape)} on {A.device}")
    if bias is not None:
        if (not bias.is_cuda or bias.dtype != torch.bfloat16 or bias.numel() != N
                or not bias.is_contiguous()):
            raise ValueError(f"bias must be a contiguous CUDA bfloat16 vector of length {N}")
    if activation not in ACTIVATIONS:
        raise ValueError(f"activation must be one of {sorted(ACTIVATIONS)}")
    fn = lib.neogemm_bf16_nt_fused_f32 if out_dtype == torch.float32 else lib.neogemm_bf16_nt_fused
    with torch.cuda.device(A.device):
        rc = fn(
            A.data_ptr(), B.data_ptr(), out.data_ptr(), M, N, K, _row_pitch("A", A),
            _row_pitch("B", B), _row_pitch("out", out), 1 if col_major else 0, float(alpha),
            float(beta), None if bias is None else bias.data_ptr(), ACTIVATIONS[activation], None,
            0, _stream_ptr(A.device))
    check(rc)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """y = x @ weight^T for x[..., K] and weight[N, K] (the layout of torch.nn.Linear): the
    operator's own layout is already x * W^T (benchmark.py:10-11,18)."""
    if x.dim() < 1:
        raise ValueError("x must have at least one dimension")
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.size(1) > 1 and x2.stride(1) != 1:
        x2 = x2.contiguous()
    y = matmul(x2, weight)
    return y.reshape(*lead, weight.size(0))


def matmul_host(A_host: torch.Tensor, B_host: torch.Tensor, C_host: torch.Tensor,
                col_major: bool = False, device: Optional[int] = None) -> torch.Tensor:
    """Product of HOST tensors through the C ABI's host entry point: copies A and B to the GPU,
    runs the kernel, copies C back and waits.  All three must be contiguous CPU bf16 tensors
    (pinned memory makes the copies asynchronous DMA)."""
    for name, t in (("A_host", A_host), ("B_host", B_host), ("C_host", C_host)):
        if t.is_cuda or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ValueError(f"{name} must be a contiguous CPU bfloat16 tensor")
    M, K = int(A_host.size(0)), int(A_host.size(1))
    N = int(B_host.size(0))
    if int(B_host.size(1)) != K or C_host.numel() != M * N:
        raise ValueError("shape mismatch between A[M,K], B[N,K] and C (M*N elements)")
    dev = torch.cuda.current_device() if device is None else device
    with torch.cuda.device(dev):
        rc = lib.neogemm_bf16_nt_host(A_host.data_ptr(), B_host.data_ptr(), C_host.data_ptr(),
                                      M, N, K, 1 if col_major else 0,
                                      _stream_ptr(torch.device("cuda", dev)))
    check(rc)
    return C_host


def workspace_bytes(M: int, N: int, K: int, col_major: bool = False) -> int:
    return int(lib.neogemm_workspace_bytes(M, N, K, 1 if col_major else 0))


def device_status() -> tuple:
    out = (ctypes.c_int * 4)()
    check(lib.neogemm_device_status(out))
    return tuple(out)


def clear_device_status() -> None:
    check(lib.neogemm_clear_device_status())


def last_config() -> dict:
    out = (ctypes.c_int * 8)()
    check(lib.neogemm_last_config(out))
    keys = ("cta_group", "block_n", "stages", "swap", "stream_k", "ctas", "tiles", "group_m")
    return dict(zip(keys, out))


def last_store_path() -> int:
    """0 regular epilogue, 1 tall tile stored as one TMA box, 2 the same with exchanged operand
    roles (neogemm_last_store_path)."""
    return int(lib.neogemm_last_store_path())


def set_override(cta_group: int = -1, block_n: int = -1, swap: int = -1, stream_k: int = -1,
                 group_m: int = -1, max_ctas: int = -1) -> None:
    """Force parts of the kernel configuration on this thread (-1 = heuristic)."""
    check(lib.neogemm_set_override(cta_group, block_n, swap, stream_k, group_m, max_ctas))


TUNING_KEYS = {"l2_hints": 0, "epilogue_wait_hint_ns": 1, "ring_wait_hint_ns": 2, "wide_tile": 3,
               "dynamic_pieces_per_tile": 4, "l2_promotion": 5, "wide_tile_prologue": 6,
               "two_ctas_per_sm": 7, "wave_pacing": 8,
               "k_direction_alternates": 9, "setup_overlap": 10,
               "two_pass_split_k": 11, "narrow_tiles": 12}


def set_tuning(key: str, value: int = -1) -> None:
    """Set one tuning knob on this thread (-1 = library default); keys: TUNING_KEYS."""
    check(lib.neogemm_set_tuning(TUNING_KEYS[key], int(value)))


__all__ = ["neoGemmV1", "neogemm", "matmul", "matmul_fused", "linear", "matmul_host", "workspace_bytes",
           "device_status", "clear_device_status", "last_config", "last_store_path", "set_override",
           "set_tuning", "NeoGemmError"]
