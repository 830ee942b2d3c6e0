"""Build recipe of the package's native code (nvcc, in-tree outputs).

``build_library()`` compiles the GEMM library ``lib/libb200_hgemm.so`` for sm_100a;
``build_driver()`` compiles the ``bin/hgemm`` benchmark driver (the C++ host surface that
mirrors the reference's ``hgemm`` executable, reference CMakeLists.txt:73-80).
Run ``python -m cuda_hgemm_b200.build`` to build both.
"""
from __future__ import annotations

import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
BIN_DIR = PKG / "bin"
LIB_SO = LIB_DIR / "libb200_hgemm.so"
COMPARE_SO = LIB_DIR / "libhgemm_compare.so"
MULTICAST_SO = LIB_DIR / "libb200_hgemm_mc.so"
MULTICAST_SRC = CSRC / "mc" / "gemm_multicast.cu"
DRIVER_BIN = BIN_DIR / "hgemm"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-std=c++17", "-O3", "-lineinfo", *ARCH_FLAGS]


def nvcc() -> str:
    return shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _up_to_date(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def _lib_sources():
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + [
        PKG.parent / "include" / "b200_hgemm.h"]


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """nvcc -> lib/libb200_hgemm.so (static cudart, no other dependency)."""
    if not force and _up_to_date(LIB_SO, _lib_sources()):
        return LIB_SO
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [nvcc(), *COMMON_FLAGS, "--shared", "-Xcompiler", "-fPIC", "-cudart", "static",
           "-o", str(LIB_SO), *[str(s) for s in sorted(CSRC.glob("*.cu"))]]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return LIB_SO


TIMELINE_SO = LIB_DIR / "libb200_hgemm_timeline.so"


def build_timeline(force: bool = False) -> Path:
    """nvcc -DB200_TIMELINE -> lib/libb200_hgemm_timeline.so: the same library with per-CTA time stamps
    (launch, set-up done, first load, first MMA, last store, exit) written to a buffer the caller hands over
    with b200_debug_set_timeline(); used by ``python -m cuda_hgemm_b200.timeline`` only."""
    if not force and _up_to_date(TIMELINE_SO, _lib_sources()):
        return TIMELINE_SO
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [nvcc(), *COMMON_FLAGS, "-DB200_TIMELINE", "--shared", "-Xcompiler", "-fPIC", "-cudart", "static",
           "-o", str(TIMELINE_SO), *[str(s) for s in sorted(CSRC.glob("*.cu"))]]
    subprocess.run(cmd, check=True)
    return TIMELINE_SO


def build_multicast(force: bool = False) -> Path | None:
    """nvcc -> lib/libb200_hgemm_mc.so, the single-GPU companion with the cluster-multicast kernel.
    Its source is not shipped to multi-GPU runs; without it there is nothing to build."""
    if not MULTICAST_SRC.exists():
        return None
    if not force and _up_to_date(MULTICAST_SO, [MULTICAST_SRC, *_lib_sources()]):
        return MULTICAST_SO
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [nvcc(), *COMMON_FLAGS, "--shared", "-Xcompiler", "-fPIC", "-cudart", "static",
           "-o", str(MULTICAST_SO), str(MULTICAST_SRC)]
    subprocess.run(cmd, check=True)
    return MULTICAST_SO


def _host_sources():
    host = CSRC / "host"
    return sorted(host.glob("*.cu")) + sorted(host.glob("*.h")) + sorted(host.glob("*.cuh"))


def build_compare(force: bool = False) -> Path:
    """nvcc -> lib/libhgemm_compare.so: the cuBLAS comparison calls behind a C ABI (links cuBLAS)."""
    src = CSRC / "host" / "cublas_tensor_op.cu"
    if not force and _up_to_date(COMPARE_SO, [src]):
        return COMPARE_SO
    LIB_DIR.mkdir(exist_ok=True)
    cmd = [nvcc(), *COMMON_FLAGS, "--shared", "-Xcompiler", "-fPIC", "-DHGEMM_COMPARE_C_ABI",
           "-o", str(COMPARE_SO), str(src), "-lcublas"]
    subprocess.run(cmd, check=True)
    return COMPARE_SO


def build_driver(force: bool = False) -> Path:
    """nvcc -> bin/hgemm, linked against the library and cuBLAS; reference kernels are loaded at run time."""
    sources = _host_sources() + _lib_sources()
    if not force and _up_to_date(DRIVER_BIN, sources):
        return DRIVER_BIN
    build_library(force=force)
    BIN_DIR.mkdir(exist_ok=True)
    host = CSRC / "host"
    cmd = [nvcc(), *COMMON_FLAGS, "-Xcompiler", "-fopenmp", "-I", str(PKG.parent / "include"), "-I", str(host),
           "-o", str(DRIVER_BIN), *[str(s) for s in sorted(host.glob("*.cu"))],
           "-L", str(LIB_DIR), "-lb200_hgemm", "-lcublas", "-ldl", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../lib"]
    subprocess.run(cmd, check=True)
    return DRIVER_BIN


def main(argv) -> int:
    force = "--force" in argv
    print("built", build_library(force=force, verbose="-v" in argv))
    mc = build_multicast(force=force)
    print("built" if mc else "no multicast source; skipped", mc or "")
    if (CSRC / "host" / "cublas_tensor_op.cu").exists():
        print("built", build_compare(force=force))
    if (CSRC / "host" / "main.cu").exists():
        print("built", build_driver(force=force))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
