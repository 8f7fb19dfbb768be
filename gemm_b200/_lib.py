"""ctypes view of libneogemm.so (the C ABI declared in include/neogemm.h).

Loading works without a GPU; any compute call then returns an error code.  There is no CPU
fallback: if the shared library is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_int64, c_size_t, c_void_p, POINTER
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libneogemm.so"

STATUS_NAMES = {
    0: "NEOGEMM_OK", 1: "NEOGEMM_ERR_BAD_ARG", 2: "NEOGEMM_ERR_UNSUPPORTED",
    3: "NEOGEMM_ERR_DESCRIPTOR", 4: "NEOGEMM_ERR_LAUNCH", 5: "NEOGEMM_ERR_DEVICE_TIMEOUT",
    6: "NEOGEMM_ERR_WORKSPACE", 7: "NEOGEMM_ERR_CUDA",
}


class NeoGemmError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, code: int, text: str):
        super().__init__(f"neogemm: {STATUS_NAMES.get(code, code)}: {text}")
        self.code = code


def _load() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m gemm_b200.build` "
            "(there is no fallback implementation)")
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.neogemm_bf16_nt.restype = c_int
    lib.neogemm_bf16_nt.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                    c_int64, c_int64, c_int64, c_int, c_void_p, c_size_t,
                                    c_void_p]
    lib.neogemm_bf16_nt_fused.restype = c_int
    lib.neogemm_bf16_nt_fused.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                          c_int64, c_int64, c_int64, c_int, ctypes.c_float,
                                          ctypes.c_float, c_void_p, c_int, c_void_p, c_size_t,
                                          c_void_p]
    lib.neogemm_bf16_nt_fused_f32.restype = c_int
    lib.neogemm_bf16_nt_fused_f32.argtypes = list(lib.neogemm_bf16_nt_fused.argtypes)
    lib.neogemm_bf16_nt_noalloc.restype = c_int
    lib.neogemm_bf16_nt_noalloc.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                                            c_int64, c_int64, c_int64, c_int64, c_int, c_void_p]
    lib.neogemm_noalloc_init.restype = c_int
    lib.neogemm_noalloc_init.argtypes = []
    lib.neogemm_noalloc_status.restype = c_int
    lib.neogemm_noalloc_status.argtypes = [POINTER(c_int), c_void_p]
    lib.neogemm_noalloc_clear_status.restype = c_int
    lib.neogemm_noalloc_clear_status.argtypes = []
    lib.neogemm_debug_wait_expiry_noalloc.restype = c_int
    lib.neogemm_debug_wait_expiry_noalloc.argtypes = [ctypes.c_uint]
    lib.neogemm_workspace_bytes.restype = c_size_t
    lib.neogemm_workspace_bytes.argtypes = [c_int64, c_int64, c_int64, c_int]
    lib.neogemm_bf16_nt_host.restype = c_int
    lib.neogemm_bf16_nt_host.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                                         c_int, c_void_p]
    lib.neogemm_device_status.restype = c_int
    lib.neogemm_device_status.argtypes = [POINTER(c_int)]
    lib.neogemm_clear_device_status.restype = c_int
    lib.neogemm_clear_device_status.argtypes = []
    lib.neogemm_status_str.restype = c_char_p
    lib.neogemm_status_str.argtypes = [c_int]
    lib.neogemm_last_config.restype = c_int
    lib.neogemm_last_config.argtypes = [POINTER(c_int)]
    lib.neogemm_last_store_path.restype = c_int
    lib.neogemm_last_store_path.argtypes = []
    lib.neogemm_set_override.restype = c_int
    lib.neogemm_set_override.argtypes = [c_int] * 6
    lib.neogemm_set_tuning.restype = c_int
    lib.neogemm_set_tuning.argtypes = [c_int, c_int]
    lib.neogemm_set_phase_timers.restype = c_int
    lib.neogemm_set_phase_timers.argtypes = [c_void_p, c_size_t]
    lib.neogemm_debug_plan.restype = c_int
    lib.neogemm_debug_plan.argtypes = [c_int64, c_int64, c_int64, c_int64, c_int, c_int,
                                       POINTER(c_int), POINTER(c_int), c_int]
    lib.neogemm_version.restype = c_int
    lib.neogemm_version.argtypes = []
    return lib


lib = _load()


def status_str(code: int) -> str:
    return lib.neogemm_status_str(int(code)).decode()


def check(code: int) -> None:
    if code != 0:
        raise NeoGemmError(code, status_str(code))
