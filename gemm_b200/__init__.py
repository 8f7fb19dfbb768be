"""B200 (sm_100a) BF16 GEMM: C = A * B^T with fp32 accumulation in tensor memory.

The operator functions live in ``gemm_b200.ops`` and are re-exported here on first use; touching
any of them loads ``libneogemm.so`` (built by ``python -m gemm_b200.build``) and raises if the
library is absent - there is no fallback implementation.  ``gemm_b200.build`` itself imports
without the library, so that it can create it.
"""
import importlib

__all__ = ["neoGemmV1", "neogemm", "matmul", "matmul_fused", "linear", "matmul_host", "workspace_bytes",
           "device_status", "clear_device_status", "last_config", "set_override", "set_tuning",
           "NeoGemmError"]


def __getattr__(name):
    if name in __all__:
        return getattr(importlib.import_module(".ops", __name__), name)
    if name in ("ops", "_lib", "shard", "inputs", "roofline", "build"):
        return importlib.import_module("." + name, __name__)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
