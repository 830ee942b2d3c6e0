"""The ``hgemm`` benchmark driver: flag handling (CPU) and, on a GPU, one full run whose log is
parsed exactly the way the reference's plot tool parses it."""
import subprocess
from pathlib import Path

import pytest

from cuda_hgemm_b200 import build

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def driver():
    if not build.DRIVER_BIN.exists():
        build.build_driver()
    return str(build.DRIVER_BIN)


def test_help_lists_the_reference_flags(driver):
    r = subprocess.run([driver, "-help"], capture_output=True, text=True)
    assert r.returncode == 0
    for flag in ("M", "N", "K", "enable_wmma", "enable_mma", "warmup_iterations", "profiling_iterations",
                 "sleep_duration", "enable_check", "cpu_procs", "gpu_rank"):
        assert f"-{flag} " in r.stderr, flag


@pytest.mark.parametrize("args", [["-bogus=1"], ["-M=abc"], ["-M=-4"], ["-K"]])
def test_bad_flags_end_the_process_with_status_1(driver, args):
    r = subprocess.run([driver, *args], capture_output=True, text=True)
    assert r.returncode == 1 and "ERROR" in r.stderr


@pytest.mark.gpu
def test_driver_run_is_parseable_by_the_reference_plot_tool(driver, cuda_device, tmp_path):
    js = tmp_path / "rows.jsonl"
    r = subprocess.run([driver, "-M=512", "-N=2048", "-K=1024", "-enable_check=true", "-warmup_iterations=2",
                        "-profiling_iterations=5", "-sleep_duration=1", "-enable_wmma=false", "-enable_mma=false",
                        f"-json={js}"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    # reference tools/performance/performance.py: lines containing 'exit' and not 'Naive', split on single spaces;
    # field 6 is the kernel name, 14 the TFLOPS, 16 the percentage in parentheses
    rows = {}
    for line in r.stderr.splitlines():
        if "exit" in line and "Naive" not in line:
            items = line.split(" ")
            rows[items[6]] = (float(items[14]), float(items[16].replace("(", "").replace(")", "").replace("%", "")))
    assert list(rows)[0] == "Cublas-Tensor-Op" and rows["Cublas-Tensor-Op"][1] == 100.0  # first kernel defines 100 %
    for name in ("B200-Tcgen05-Auto", "B200-Tcgen05-1Cta", "B200-Tcgen05-2Cta", "B200-Tcgen05-SplitK",
                 "B200-Tcgen05-StreamK"):
        assert name in rows and rows[name][0] > 1.0
    assert "check vs FP32 host GEMM" in r.stderr and "FAIL" not in r.stderr
    assert "Done" in r.stderr.splitlines()[-1]
    import json

    parsed = [json.loads(x) for x in js.read_text().splitlines()]
    ours = [p for p in parsed if p["kernel"].startswith("B200-")]
    assert ours and all(p["checked"] and p["pass"] and 0 <= p["max_rel_err"] < 2e-3 for p in ours)


@pytest.mark.gpu
def test_driver_runs_the_reference_kernels_when_their_library_is_present(driver, cuda_device):
    ref = ROOT / "oracle" / "_ref" / "libcuda_hgemm_ref.so"
    if not ref.exists():
        pytest.skip("the reference's kernels were not built (no reference checkout at build time)")
    r = subprocess.run([driver, "-M=256", "-N=256", "-K=256", "-enable_check=true", "-warmup_iterations=1",
                        "-profiling_iterations=2", "-sleep_duration=1", "-enable_variants=false", f"-ref_lib={ref}"],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    for name in ("Wmma-Padding", "Wmma-Async-Stage3", "Mma-Permuted", "Mma-Async-Stage4", "B200-Tcgen05-Auto"):
        assert f"{name} exit" in r.stderr
