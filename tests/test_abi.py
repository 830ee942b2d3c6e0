"""The C-ABI library loads and exports every symbol include/b200_hgemm.h declares; argument
checking answers before any device is touched. CPU only: no compute call is made."""
import ctypes
import re
from pathlib import Path

import pytest

from cuda_hgemm_b200 import _native

HEADER = Path(__file__).resolve().parent.parent / "include" / "b200_hgemm.h"


def declared_functions():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_functions() == sorted(_native.EXPORTED_SYMBOLS)


def test_every_declared_symbol_is_exported(native_lib):
    for name in declared_functions():
        assert hasattr(native_lib, name), f"{name} is declared in the header but not exported"


def test_version_and_status_strings(native_lib):
    assert b"sm_100a" in native_lib.b200_hgemm_version()
    seen = set()
    for code in (0, -1, -2, -3, -4, -5, -6, -7, -8):
        s = native_lib.b200_hgemm_status_string(code)
        assert s and s not in seen
        seen.add(s)
    assert native_lib.b200_hgemm_status_string(-99) == b"unknown status"


def test_argument_errors_come_before_any_device_work(native_lib):
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    for fn in (native_lib.b200_hgemm, native_lib.b200_hgemm_cta1, native_lib.b200_hgemm_cta2,
               native_lib.b200_hgemm_splitk, native_lib.b200_hgemm_streamk, native_lib.b200_hgemm_simt):
        assert fn(None, p, p, 8, 8, 8, None) == _native.ERR_INVALID_ARG
        assert fn(p, p, p, 0, 8, 8, None) == _native.ERR_INVALID_ARG
        assert fn(p, p, p, 8, 8, 0, None) == _native.ERR_INVALID_ARG
    assert native_lib.b200_hgemm_ex(p, p, p, 8, 8, 8, None, None) == _native.ERR_INVALID_ARG
    assert native_lib.b200_hgemm_host(None, p, p, 8, 8, 8) == _native.ERR_INVALID_ARG


def test_no_silent_fallback_without_a_gpu(native_lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present; the no-device answer cannot be observed")
    buf = ctypes.create_string_buffer(4096)
    p = (ctypes.addressof(buf) + 15) & ~15
    # valid arguments, no device: the call must fail loudly, never compute on the host
    assert native_lib.b200_hgemm(p, p, p, 8, 8, 8, None) in (_native.ERR_CUDA, _native.ERR_NO_SM100)
    with pytest.raises(_native.HgemmError):
        _native.check(native_lib.b200_hgemm(p, p, p, 8, 8, 8, None))


def test_missing_library_raises(monkeypatch, tmp_path):
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _native.load()


def test_descriptor_encoders(native_lib):
    # instruction descriptor: D=F32 (bit 4), A/B=F16 K-major (zeros), N>>3 at bit 17, M>>4 at bit 24
    assert native_lib.b200_debug_idesc(128, 256) == (1 << 4) | (32 << 17) | (8 << 24)
    assert native_lib.b200_debug_idesc(256, 256) == (1 << 4) | (32 << 17) | (16 << 24)
    assert native_lib.b200_debug_idesc(128, 64) == (1 << 4) | (8 << 17) | (8 << 24)
    # shared-memory descriptor: addr>>4 | LBO 1 | SBO 1024>>4 | version 1 | 128-byte swizzle (2)
    d = native_lib.b200_debug_smem_desc(0x12400)
    assert d & 0x3FFF == 0x12400 >> 4
    assert (d >> 16) & 0x3FFF == 1
    assert (d >> 32) & 0x3FFF == 64
    assert (d >> 46) & 0x3 == 1
    assert (d >> 61) & 0x7 == 2
    # stepping 16 halves (32 bytes) along K adds 2 to the address field
    assert native_lib.b200_debug_smem_desc(0x12400 + 32) - d == 2


def test_plan_selection_covers_the_benchmark_shapes(native_lib):
    from cuda_hgemm_b200 import api

    # long k, many tiles: 256 x 256 outputs per CTA (pairs, or groups of four with the multicast companion)
    big = api.select_plan_untuned(8192, 8192, 8192)
    assert big.variant in (_native.VARIANT_CTA2, _native.VARIANT_CTA2_MCAST) and big.bn == 512
    # short k: the drain of a full tensor memory would show; 128 x 256 per CTA with two accumulator sets
    short_k = api.select_plan_untuned(4096, 4096, 1024)
    assert short_k.variant == _native.VARIANT_CTA2 and short_k.bn == 256
    # a last wave that the larger tiles would leave emptier
    assert api.select_plan_untuned(3584, 3584, 3584).bn == 256
    # decode shapes: the kernel for a short A; whole k-ranges at N = 14336 (112 column tiles), cut at N = 4096
    wide = api.select_plan_untuned(16, 14336, 4096)
    assert wide.variant == _native.VARIANT_SKINNY and wide.bn == 16
    assert api.workspace_bytes(16, 14336, 4096, wide) == 0
    skinny = api.select_plan_untuned(48, 4096, 14336)
    assert skinny.variant == _native.VARIANT_SKINNY and skinny.bn == 64
    assert api.workspace_bytes(48, 4096, 14336, skinny) == 0  # four k-ranges per tile: one cluster, summed on chip
    through_workspace = api.select_plan_untuned(48, 4096, 14336)
    through_workspace.grid = 2
    assert api.workspace_bytes(48, 4096, 14336, through_workspace) > 0
    # 16 column tiles would make nine k-ranges: four of them in one cluster instead (64 of 148 SMs)
    assert api.workspace_bytes(16, 2048, 8192, api.select_plan_untuned(16, 2048, 8192)) == 0
    # four column tiles: 16 CTAs would be too few, 37 k-ranges go through the workspace
    assert api.workspace_bytes(16, 512, 8192, api.select_plan_untuned(16, 512, 8192)) > 0
    # 65 ... 128 rows against a large B: the same kernel on CTA pairs; single CTAs with k cut where the column tiles are few
    wide128 = api.select_plan_untuned(128, 14336, 4096)
    assert (wide128.variant, wide128.bn) == (_native.VARIANT_SKINNY_PAIR, 128)
    assert api.workspace_bytes(128, 14336, 4096, wide128) == 0
    mid = api.select_plan_untuned(96, 4096, 14336)  # single CTAs, so that the four k-ranges fit a cluster of four
    assert (mid.variant, mid.bn) == (_native.VARIANT_SKINNY, 128) and api.workspace_bytes(96, 4096, 14336, mid) == 0
    # small problems of that height keep the 128-row tiles or k-ranges over them
    assert api.select_plan_untuned(100, 512, 4096).variant in (_native.VARIANT_CTA1, _native.VARIANT_STREAMK)
    assert api.workspace_bytes(8192, 8192, 8192, big) == 0
    odd = api.select_plan_untuned(48, 40, 100)
    assert odd.variant == _native.VARIANT_SIMT  # K % 8 != 0: no TMA row pitch
    ragged_n = api.select_plan_untuned(512, 1001, 512)
    assert ragged_n.tma_store == 0


def test_tuned_plan_table_overrides_the_rules(native_lib, tmp_path):
    from cuda_hgemm_b200 import api

    table = tmp_path / "plan_table.txt"
    table.write_text("# a comment line\n"
                     "2304 2304 2304 1 128 0 4 1   # pairs on 256 x 128, bands of 4\n"
                     "40 4096 4096 5 32 0 0 1      # short-A tile of 32 rows for 40 rows: cannot be served\n"
                     "not a plan line\n"
                     "512 512 512 2 64 7 0 1\n")
    try:
        assert api.load_plan_table(table) == 3
        tuned = api.select_plan(2304, 2304, 2304)
        assert (tuned.variant, tuned.bn, tuned.group_m) == (_native.VARIANT_CTA2, 128, 4)
        assert (api.select_plan(512, 512, 512).variant, api.select_plan(512, 512, 512).parts) == (_native.VARIANT_STREAMK, 7)
        # the rules still answer when asked directly, and for every shape the table does not list or cannot serve
        rules = api.select_plan_untuned(2304, 2304, 2304)
        assert (rules.variant, rules.bn) != (tuned.variant, tuned.bn)
        assert api.select_plan(2304, 2304, 2305).variant == api.select_plan_untuned(2304, 2304, 2305).variant
        unserved = api.select_plan(40, 4096, 4096)
        assert (unserved.variant, unserved.bn) == (_native.VARIANT_SKINNY, 64)
        with pytest.raises(_native.HgemmError):
            api.load_plan_table(tmp_path / "missing.txt")
    finally:
        assert api.load_plan_table(None) == 0
    assert api.select_plan(2304, 2304, 2304).bn == api.select_plan_untuned(2304, 2304, 2304).bn



def test_every_plan_the_rules_pick_is_one_the_kernels_can_serve(native_lib):
    """Seeded shapes over six orders of magnitude: the plan's fields stay inside what run_plan accepts."""
    import numpy as np

    from cuda_hgemm_b200 import api

    rng = np.random.default_rng(99)
    V = _native
    seen = set()
    for _ in range(3000):
        M, N, K = (int(2 ** rng.uniform(0, 15)) for _ in range(3))
        if rng.random() < 0.5:
            K = max(8, K // 8 * 8)
        if rng.random() < 0.5:
            N = max(8, N // 8 * 8)
        p = api.select_plan_untuned(M, N, K)
        seen.add((p.variant, p.bn))
        what = f"{(M, N, K)} -> {p.as_dict()}"
        if K % 8 != 0:
            assert p.variant == V.VARIANT_SIMT, what
            continue
        assert p.variant in (V.VARIANT_CTA1, V.VARIANT_CTA2, V.VARIANT_STREAMK, V.VARIANT_CTA2_MCAST, V.VARIANT_SKINNY,
                             V.VARIANT_SKINNY_PAIR), what
        assert p.parts == 0 and p.grid == 0 and p.group_m == 0, what
        if p.variant == V.VARIANT_SKINNY and p.bn == 128:
            # 65 ... 128 rows on single CTAs only where k would be cut into three or more ranges (four, one cluster per tile)
            assert 64 < M <= 128 and N >= 2048 and K >= 1024 and 148 // -(-N // 128) >= 3, what
            continue
        if p.variant == V.VARIANT_SKINNY:
            assert M <= 64 and p.bn in (16, 32, 64) and M <= p.bn and (p.bn == 16 or M > p.bn // 2), what
            continue
        if p.variant == V.VARIANT_SKINNY_PAIR:
            assert 64 < M <= 128 and p.bn == 128 and N >= 2048 and K >= 1024, what
            continue
        assert M > 64, what
        assert p.tma_store == (1 if N % 8 == 0 else 0), what
        if p.variant == V.VARIANT_CTA1:
            assert p.bn in (64, 128, 256), what
        elif p.variant == V.VARIANT_STREAMK:
            assert p.bn in (64, 128, 256) and -(-K // 64) >= 8, what
        elif p.variant == V.VARIANT_CTA2:
            assert p.bn in (192, 224, 256, 288, 320, 512) and M > 128, what
        if p.bn == 512:  # 256 x 256 outputs per CTA: TMA stores only, long k, long runs
            assert N % 8 == 0 and -(-K // 64) >= 24 and 2.0 * M * N * K >= 2.0 * 4096 ** 3, what
    # the draw reaches every family
    assert {V.VARIANT_SIMT, V.VARIANT_CTA1, V.VARIANT_CTA2, V.VARIANT_STREAMK, V.VARIANT_SKINNY} <= {v for v, _ in seen}


def test_workspace_sizes_callers_can_rely_on(native_lib):
    """b200_hgemm_workspace_bytes for the kernels that cut k (a caller sizing its own workspace uses these)."""
    from cuda_hgemm_b200 import api

    def plan(variant, bn, parts=0, grid=0):
        p = _native.Plan()
        p.variant, p.bn, p.parts, p.tma_store, p.grid = variant, bn, parts, 1, grid
        return p

    header = 64 * 1024
    # stream-k: two FP32 partial-tile slots of 128 x bn per k-range, one k-range per SM of a 148-SM part by default
    assert api.workspace_bytes(96, 4096, 14336, plan(_native.VARIANT_STREAMK, 128)) == header + 148 * 2 * 128 * 128 * 4
    assert api.workspace_bytes(96, 4096, 14336, plan(_native.VARIANT_STREAMK, 256, parts=40)) == header + 40 * 2 * 128 * 256 * 4
    # never more k-ranges than (tile, stage) units: 2 tiles x 2 stages of two k-blocks each
    assert api.workspace_bytes(128, 256, 256, plan(_native.VARIANT_STREAMK, 128)) == header + 4 * 2 * 128 * 128 * 4
    assert api.workspace_bytes(128, 256, 256, plan(_native.VARIANT_HYBRID, 128)) == header + 4 * 2 * 128 * 128 * 4
    # short A, k cut (32 column tiles -> 4 k-ranges) and summed through the workspace (plan.grid = 2): k-ranges x tile
    # height x padded N floats; nothing when the k-ranges are summed inside clusters (the library's choice up to four
    # CTAs per cluster, or plan.grid = 1 up to eight) or when k is whole
    assert api.workspace_bytes(48, 4096, 14336, plan(_native.VARIANT_SKINNY, 64, grid=2)) == 4 * 64 * 4096 * 4
    assert api.workspace_bytes(48, 4100, 14336, plan(_native.VARIANT_SKINNY, 64, parts=3, grid=2)) == 3 * 64 * 4128 * 4
    assert api.workspace_bytes(48, 4096, 14336, plan(_native.VARIANT_SKINNY, 64)) == 0
    assert api.workspace_bytes(48, 4096, 14336, plan(_native.VARIANT_SKINNY, 64, parts=8, grid=1)) == 0
    assert api.workspace_bytes(48, 4096, 14336, plan(_native.VARIANT_SKINNY, 64, parts=8)) == 8 * 64 * 4096 * 4
    assert api.workspace_bytes(48, 4096, 14336, plan(_native.VARIANT_SKINNY_PAIR, 64)) == 4 * 64 * 4096 * 4  # clusters of eight
    assert api.workspace_bytes(48, 4096, 14336, plan(_native.VARIANT_SKINNY_PAIR, 64, parts=2)) == 0
    assert api.workspace_bytes(16, 14336, 4096, plan(_native.VARIANT_SKINNY, 16)) == 0
    # whole-tile kernels need none
    for variant, bn in ((_native.VARIANT_CTA1, 256), (_native.VARIANT_CTA2, 512), (_native.VARIANT_CTA2_MCAST, 512)):
        assert api.workspace_bytes(8192, 8192, 8192, plan(variant, bn)) == 0


def test_short_a_k_slices_are_never_empty(native_lib):
    """The short-A kernel gives every CTA one k-range; the launcher must never hand out an empty one.
    The slice count is read back from the workspace size (slices x tile height x padded N floats)."""
    import numpy as np

    from cuda_hgemm_b200 import api

    rng = np.random.default_rng(7)
    for _ in range(2000):
        N = int(rng.integers(1, 20000))
        K = int(rng.integers(1, 4000)) * 8
        bn = int(rng.choice([16, 32, 64]))
        parts = int(rng.choice([0, 0, 1, 2, 3, 5, 8, 37, 300]))
        p = _native.Plan()
        p.variant, p.bn, p.parts = _native.VARIANT_SKINNY, bn, parts
        n_pad = (N + 31) // 32 * 32
        ws = api.workspace_bytes(8, N, K, p)
        assert ws % (bn * n_pad * 4) == 0
        slices = ws // (bn * n_pad * 4) or 1
        k_blocks = -(-K // 64)
        per = -(-k_blocks // slices)
        assert 1 <= slices <= k_blocks, (N, K, bn, parts, slices)
        assert (slices - 1) * per < k_blocks, f"slice {slices - 1} of {slices} would be empty: {(N, K, bn, parts)}"
        if parts == 0 and slices > 1:
            assert per >= 8 and slices * -(-N // 128) <= 148, (N, K, slices)


def test_public_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 (and as C++) on its own."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    root = Path(__file__).resolve().parents[1]
    src = tmp_path / "include_test.c"
    src.write_text('#include "b200_hgemm.h"\n'
                   "int main(void) { b200_hgemm_plan p; b200_hgemm_epilogue e; b200_mg *mg = 0; (void)p; (void)e; (void)mg; "
                   "return b200_hgemm_status_string(0) != 0; }\n")
    for args in (["-std=c99", "-pedantic"], ["-x", "c++", "-std=c++11"]):
        subprocess.run([gcc, *args, "-Wall", "-Wextra", "-Werror", "-fsyntax-only", f"-I{root / 'include'}", str(src)], check=True)


def test_plan_supported_knows_the_cluster_limit_of_the_short_a_kernels(native_lib):
    """plan.grid = 1 asks for the k-ranges of a tile in one cluster: at most eight CTAs (four k-ranges for pairs)."""
    import ctypes

    def plan(variant, bn, parts, grid):
        p = _native.Plan()
        p.variant, p.bn, p.parts, p.tma_store, p.grid = variant, bn, parts, 1, grid
        return p

    lib = native_lib
    ok = lambda p: lib.b200_hgemm_plan_supported(16, 4096, 14336, ctypes.byref(p))  # noqa: E731
    assert ok(plan(_native.VARIANT_SKINNY, 16, 8, 1)) == _native.OK
    assert ok(plan(_native.VARIANT_SKINNY, 16, 9, 1)) == _native.ERR_UNSUPPORTED
    assert ok(plan(_native.VARIANT_SKINNY, 16, 9, 2)) == _native.OK
    assert ok(plan(_native.VARIANT_SKINNY, 16, 9, 0)) == _native.OK       # the library's choice: through the workspace
    assert ok(plan(_native.VARIANT_SKINNY_PAIR, 16, 4, 1)) == _native.OK
    assert ok(plan(_native.VARIANT_SKINNY_PAIR, 16, 5, 1)) == _native.ERR_UNSUPPORTED
    assert ok(plan(_native.VARIANT_SKINNY, 16, 4, 3)) == _native.ERR_UNSUPPORTED  # grid names nothing beyond 2 here
