"""CPU: the C-ABI library loads without a GPU, exports every symbol the header declares, and
rejects bad arguments with the documented codes before touching a device."""
import ctypes
import os
import re

import pytest
import torch

from gemm_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "neogemm.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(neogemm_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for n in ("neogemm_bf16_nt", "neogemm_bf16_nt_host", "neogemm_workspace_bytes",
              "neogemm_status_str", "neogemm_device_status", "neogemm_last_config"):
        assert n in names


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in neogemm.h but not exported"


def test_status_strings():
    assert _lib.status_str(0) == "ok"
    for code in range(1, 8):
        s = _lib.status_str(code)
        assert s and s != "unknown status"
    assert _lib.status_str(99) == "unknown status"
    assert _lib.lib.neogemm_version() >= 100


def test_argument_validation_needs_no_device():
    f = _lib.lib.neogemm_bf16_nt
    buf = torch.zeros(64 * 64, dtype=torch.bfloat16)
    p = buf.data_ptr()
    assert p % 16 == 0
    # negative size
    assert f(p, p, p, -1, 8, 8, 8, 8, 8, 0, None, 0, None) == 1
    # null C
    assert f(p, p, None, 8, 8, 8, 8, 8, 8, 0, None, 0, None) == 1
    # null A with K > 0
    assert f(None, p, p, 8, 8, 8, 8, 8, 8, 0, None, 0, None) == 1
    # lda < K
    assert f(p, p, p, 8, 8, 16, 8, 16, 8, 0, None, 0, None) == 1
    # ldc shorter than the stored row
    assert f(p, p, p, 8, 16, 8, 8, 8, 8, 0, None, 0, None) == 1
    assert f(p, p, p, 16, 8, 8, 8, 8, 8, 1, None, 0, None) == 1
    # K not a multiple of 8 -> unsupported
    assert f(p, p, p, 8, 8, 12, 16, 16, 8, 0, None, 0, None) == 2
    # lda not a multiple of 8
    assert f(p, p, p, 8, 8, 8, 12, 8, 8, 0, None, 0, None) == 2
    # misaligned A
    assert f(p + 2, p, p, 8, 8, 8, 8, 8, 8, 0, None, 0, None) == 2
    # empty problems are no-ops even without a device
    assert f(None, None, None, 0, 8, 8, 8, 8, 8, 0, None, 0, None) == 0
    assert f(None, None, None, 8, 0, 8, 8, 8, 8, 0, None, 0, None) == 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU behaviour")
def test_compute_calls_fail_loudly_without_a_gpu():
    buf = torch.zeros(64 * 64, dtype=torch.bfloat16)
    p = buf.data_ptr()
    rc = _lib.lib.neogemm_bf16_nt(p, p, p, 64, 64, 64, 64, 64, 64, 0, None, 0, None)
    assert rc != 0, "a valid problem must not 'succeed' on a machine without a GPU"
    rc = _lib.lib.neogemm_bf16_nt_host(p, p, p, 64, 64, 64, 0, None)
    assert rc != 0
    assert _lib.lib.neogemm_workspace_bytes(16, 28672, 8192, 0) == 0
    out = (ctypes.c_int * 4)()
    assert _lib.lib.neogemm_device_status(out) != 0


def test_override_rejects_nonsense():
    assert _lib.lib.neogemm_set_override(3, -1, -1, -1, -1, -1) == 1
    assert _lib.lib.neogemm_set_override(-1, 48, -1, -1, -1, -1) == 1
    assert _lib.lib.neogemm_set_override(-1, -1, -1, -1, -1, -1) == 0


def test_python_wrapper_rejects_cpu_tensors():
    from gemm_b200 import ops
    a = torch.zeros(8, 8, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        ops.matmul(a, a)
    with pytest.raises(ValueError):
        ops.neoGemmV1(a, a, torch.zeros(8, 8, dtype=torch.bfloat16))
