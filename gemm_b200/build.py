"""Build steps for the native parts: the CUDA library (nvcc), the torch binding (g++ through
setup.py) and the test-only CPU oracle (gcc).

The reference builds one torch CUDAExtension from a single .cu that includes torch headers
(setup.py:4-24).  Here the kernels and the C-ABI launcher are compiled by nvcc alone into
``gemm_b200/libneogemm.so`` (seconds), and only the thin binding (csrc/binding.cpp) sees torch.
Everything is built in-tree so that the shared objects travel with the source directory.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
ROOT = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_PATH = PKG_DIR / "libneogemm.so"
ORACLE_DIR = ROOT / "oracle"
ORACLE_LIB = ORACLE_DIR / "liboracle.so"

# Explicit -gencode: plain -arch=sm_100a would also emit generic compute_100 PTX, for which ptxas
# rejects every tcgen05 instruction.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "-DNDEBUG",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return nvcc


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def library_sources():
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [ROOT / "include" / "neogemm.h"]


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """nvcc: csrc/*.cu -> gemm_b200/libneogemm.so for sm_100a."""
    srcs = library_sources()
    if not force and _newer(LIB_PATH, srcs):
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_FLAGS, "-shared", "-o", str(LIB_PATH)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(p) for p in sorted(CSRC.glob("*.cu"))]
    subprocess.run(cmd, check=True, cwd=str(ROOT))
    return LIB_PATH


def build_oracle(force: bool = False) -> Path:
    """gcc: oracle/gemm_oracle.c -> oracle/liboracle.so (test infrastructure)."""
    src = ORACLE_DIR / "gemm_oracle.c"
    if not force and _newer(ORACLE_LIB, [src]):
        return ORACLE_LIB
    subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-o", str(ORACLE_LIB), str(src)], check=True)
    return ORACLE_LIB


def extension_path():
    hits = sorted(ROOT.glob("neoGEMM*.so"))
    return hits[0] if hits else None


def build_extension(force: bool = False) -> Path:
    """setup.py build_ext --inplace: csrc/binding.cpp -> neoGEMM.*.so at the repository root."""
    ext = extension_path()
    srcs = [CSRC / "binding.cpp", ROOT / "include" / "neogemm.h", ROOT / "setup.py"]
    if not force and ext is not None and _newer(ext, srcs) and _newer(ext, [LIB_PATH]):
        return ext
    subprocess.run([sys.executable, "setup.py", "-q", "build_ext", "--inplace"], check=True,
                   cwd=str(ROOT))
    ext = extension_path()
    if ext is None:
        raise RuntimeError("setup.py did not produce the neoGEMM extension")
    return ext


def build_all(force: bool = False) -> None:
    build_library(force)
    build_extension(force)
    build_oracle(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(LIB_PATH, extension_path(), ORACLE_LIB)
