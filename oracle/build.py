"""Build recipe for the checker libraries (test infrastructure, not the product).

* ``libhgemm_oracle.so``  -- the CPU restatement in ``hgemm_oracle.c`` (gcc, OpenMP).
* ``_ref/libcuda_hgemm_ref.so`` -- the reference project's own kernels, compiled unmodified
  from where its sources lie (never copied into this repository) for sm_100a, with the flags of
  its release build (reference CMakeLists.txt:49,53 with the architecture swapped). It is only
  built when the reference checkout is present; the result is git-ignored.

Usage: ``python oracle/build.py [oracle] [ref]`` (default: both, the second only if possible).
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
ORACLE_SO = HERE / "libhgemm_oracle.so"
REF_DIR = HERE / "_ref"
REF_SO = REF_DIR / "libcuda_hgemm_ref.so"
# the reference checkout: CUDA_HGEMM_REFERENCE, else a directory named "reference" beside this repository
REFERENCE_ROOT = Path(os.environ.get("CUDA_HGEMM_REFERENCE") or HERE.parent.parent / "reference")

# reference kernels: entry point -> log name used by its driver (reference src/main.cu:100-123)
REF_KERNELS = {
    "cublasTensorOp": "Cublas-Tensor-Op",
    "simtNaive": "Simt-Naive",
    "wmmaNaive": "Wmma-Naive",
    "wmmaBase": "Wmma-Base",
    "wmmaPadding": "Wmma-Padding",
    "wmmaAsync": "Wmma-Async",
    "wmmaAsyncPg2s": "Wmma-Async-Pg2s",
    "wmmaAsyncPg2sPs2r": "Wmma-Async-Pg2s-Ps2r",
    "wmmaAsyncStage2": "Wmma-Async-Stage2",
    "wmmaAsyncStage3": "Wmma-Async-Stage3",
    "mmaNaive": "Mma-Naive",
    "mmaBase": "Mma-Base",
    "mmaPermuted": "Mma-Permuted",
    "mmaAsync": "Mma-Async",
    "mmaAsyncPg2s": "Mma-Async-Pg2s",
    "mmaAsyncPg2sPs2r": "Mma-Async-Pg2s-Ps2r",
    "mmaAsyncStage2": "Mma-Async-Stage2",
    "mmaAsyncStage3": "Mma-Async-Stage3",
    "mmaAsyncStage4": "Mma-Async-Stage4",
}


def mangled(entry: str) -> str:
    """Itanium-mangled name of ``void entry(half*, half*, half*, size_t, size_t, size_t)``."""
    return f"_Z{len(entry)}{entry}P6__halfS0_S0_mmm"


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def build_oracle(force: bool = False) -> Path:
    src = HERE / "hgemm_oracle.c"
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    cmd = ["gcc", "-O3", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-mavx2", "-mfma", "-mf16c",
           "-fno-math-errno", "-o", str(ORACLE_SO), str(src), "-lm"]
    subprocess.run(cmd, check=True)
    return ORACLE_SO


def reference_available() -> bool:
    return (REFERENCE_ROOT / "src" / "mma" / "mma_async_stage4.cu").exists()


def build_ref(force: bool = False) -> Path | None:
    """Compile the reference's kernels where they lie. Returns None when there is no checkout."""
    if not reference_available():
        return REF_SO if REF_SO.exists() else None
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    src_root = REFERENCE_ROOT / "src"
    sources = sorted(src_root.glob("mma/*.cu")) + sorted(src_root.glob("wmma/*.cu")) + [
        src_root / "simt_naive.cu", src_root / "cublas_tensor_op.cu"]
    if not force and _newer(REF_SO, sources):
        return REF_SO
    REF_DIR.mkdir(exist_ok=True)
    obj_dir = REF_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    flags = ["-std=c++14", "-O3", "--use_fast_math", "--expt-relaxed-constexpr", "-Xcompiler", "-fopenmp",
             "-Xcompiler", "-fPIC", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
             "-I", str(src_root / "common")]

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        subprocess.run([nvcc, *flags, "-c", str(src), "-o", str(obj)], check=True,
                       stdout=subprocess.DEVNULL, stderr=subprocess.PIPE)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objs = list(pool.map(compile_one, sources))
    subprocess.run([nvcc, "-shared", "-o", str(REF_SO), *map(str, objs), "-lcublas", "-Xcompiler", "-fopenmp"],
                   check=True)
    shutil.rmtree(obj_dir, ignore_errors=True)
    return REF_SO


def main(argv) -> int:
    what = set(argv) or {"oracle", "ref"}
    if "oracle" in what:
        print("built", build_oracle(force=True))
    if "ref" in what:
        out = build_ref(force=True)
        print("built" if out else "reference checkout absent; skipped", out or "")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
