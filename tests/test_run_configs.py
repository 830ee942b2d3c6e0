"""The configuration runner builds driver command lines; they must only use flags the driver defines."""
import re
from pathlib import Path

from cuda_hgemm_b200 import run_configs

MAIN_CU = Path(__file__).resolve().parents[1] / "cuda_hgemm_b200" / "csrc" / "host" / "main.cu"


def driver_flags():
    return set(re.findall(r"DEFINE_\w+\((\w+),", MAIN_CU.read_text()))


def test_every_flag_used_is_defined_by_the_driver(tmp_path):
    defined = driver_flags()
    assert {"M", "N", "K", "dist", "l2_rotate", "ref_lib", "json"} <= defined
    for config in run_configs.CONFIGS:
        for M, N, K, extra in run_configs.shapes_of(config):
            cmd = run_configs.command(Path("hgemm"), tmp_path, M, N, K, extra, "ref.so", 3, 10)
            for arg in cmd[1:]:
                name = arg.lstrip("-").split("=", 1)[0]
                assert name in defined, f"{arg} in configuration {config} is not a driver flag"


def test_configurations_hold_the_benchmark_shapes():
    assert run_configs.shapes_of("small")[0][:3] == (256, 256, 256)
    squares = run_configs.shapes_of("squares")
    assert len(squares) == 64 and squares[0][:3] == (256, 256, 256) and squares[-1][:3] == (16384, 16384, 16384)
    decode = {s[:3] for s in run_configs.shapes_of("decode")}
    assert decode == {(m, n, k) for m in (16, 32, 64, 128) for n, k in ((14336, 4096), (4096, 14336))}
    assert run_configs.shapes_of("prefill")[0][:3] == (8192, 28672, 8192)


def test_reference_kernels_only_on_shapes_they_accept(tmp_path, capsys):
    # the reference's tuned kernels need M % 256 = N % 128 = K % 32 = 0: the decode shapes run without them
    with_ref = run_configs.command(Path("hgemm"), tmp_path, 8192, 28672, 8192, [], "ref.so", 3, 10)
    without = run_configs.command(Path("hgemm"), tmp_path, 16, 14336, 4096, [], "ref.so", 3, 10)
    assert "-ref_lib=ref.so" in with_ref and "-ref_lib=ref.so" not in without
    assert "-enable_wmma=false" in without and "-enable_mma=false" in without
    assert run_configs.main(["--out", str(tmp_path), "--configs", "small,prefill", "--dry-run"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2 and "-M=256" in lines[0] and "-N=28672" in lines[1]
