"""The tool that regenerates ``profiles/``: its capture table keeps to small captures, and its CSV reader and
summary writer work on a recorded sample of ncu's output format. No GPU and no ncu run here."""
from pathlib import Path

from cuda_hgemm_b200 import profile

SAMPLE = '''==PROF== Connected to process 1234
==PROF== Disconnected from process 1234
"ID","Process ID","Process Name","Host Name","Kernel Name","Context","Stream","Block Size","Grid Size","Device","CC","Section Name","Metric Name","Metric Unit","Metric Value"
"0","1234","python","box","void b200::hgemm_skinny_kernel<16, 6, 2, 1, 0>(b200::SkinnyParams)","1","7","(192, 1, 1)","(138, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_read.sum","Mbyte","117.61"
"0","1234","python","box","void b200::hgemm_skinny_kernel<16, 6, 2, 1, 0>(b200::SkinnyParams)","1","7","(192, 1, 1)","(138, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_write.sum","Mbyte","3.90"
"0","1234","python","box","void b200::hgemm_skinny_kernel<16, 6, 2, 1, 0>(b200::SkinnyParams)","1","7","(192, 1, 1)","(138, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","us","25.12"
"1","1234","python","box","void b200::hgemm_skinny_kernel<16, 6, 2, 1, 0>(b200::SkinnyParams)","1","7","(192, 1, 1)","(138, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_read.sum","Mbyte","117.59"
"1","1234","python","box","void b200::hgemm_skinny_kernel<16, 6, 2, 1, 0>(b200::SkinnyParams)","1","7","(192, 1, 1)","(138, 1, 1)","0","10.0","Command line profiler metrics","dram__bytes_write.sum","Mbyte","4,10"
"1","1234","python","box","void b200::hgemm_skinny_kernel<16, 6, 2, 1, 0>(b200::SkinnyParams)","1","7","(192, 1, 1)","(138, 1, 1)","0","10.0","Command line profiler metrics","gpu__time_duration.sum","us","24.90"
'''


def test_captures_stay_small():
    for name, (title, target, regex, skip, count, shape) in profile.CAPTURES.items():
        assert title and target
        if regex is None:
            continue  # the launch list: gpu__time_duration.sum alone, one pass per launch
        assert count <= 3, name
        assert shape is not None
        M, N, K = shape
        assert 2 * (M * K + N * K + M * N) <= 4e9, f"{name}: more than a few GB of operands"
    # every target is a committed module or bench.py
    for _, (_, target, *_rest) in profile.CAPTURES.items():
        assert target[1:3] == ["-m", "cuda_hgemm_b200.profile_target"] or target[1] == "bench.py"


def test_csv_reader_and_summary(tmp_path):
    path = tmp_path / "sample.csv"
    path.write_text(SAMPLE)
    launches = profile.parse_ncu_csv(path)
    assert len(launches) == 2 and all("hgemm_skinny_kernel" in k for k, _ in launches)
    assert launches[0][1]["dram__bytes_read.sum"] == (117.61, "Mbyte")
    assert launches[1][1]["dram__bytes_write.sum"] == (410.0, "Mbyte")  # thousands separators are dropped
    text = profile.summarise_capture("x", "title", ["python", "-m", "t"], ["ncu", "python", "-m", "t"], launches[:1], (16, 14336, 4096))
    assert "121.5 MB per launch = 1.03 x algorithmic" in text
    assert "ncu python -m t" in text and "25.1" in text
    listing = profile.summarise_launch_list("bench", ["python", "bench.py"], ["ncu", "python", "bench.py"], launches)
    assert "| 2 |" in listing and "100.0 %" in listing


def test_units():
    assert profile.to_ns(2.0, "ms") == 2e6 and profile.to_ns(3.0, "us") == 3e3
    assert profile.to_bytes(1.5, "Gbyte") == 1.5e9
