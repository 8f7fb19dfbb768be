"""B200 (sm_100a) BF16 GEMM: C = A * B^T with fp32 accumulation in tensor memory.

Importing the package loads ``libneogemm.so`` (built by ``python -m gemm_b200.build``); it fails
loudly if the library is absent - there is no fallback implementation.
"""
from .ops import (NeoGemmError, clear_device_status, device_status, last_config, linear, matmul,
                  matmul_host, neoGemmV1, neogemm, set_override, workspace_bytes)

__all__ = ["neoGemmV1", "neogemm", "matmul", "linear", "matmul_host", "workspace_bytes",
           "device_status", "clear_device_status", "last_config", "set_override", "NeoGemmError"]
