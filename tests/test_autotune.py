"""The autotuner's host-side logic (which plans it times, what it writes); the timing itself needs a GPU."""
from cuda_hgemm_b200 import _native, autotune


def keys(M, N, K):
    return {(p.variant, p.bn) for p in autotune.candidate_plans(M, N, K)}


def test_candidates_follow_the_shape():
    # a large square: single-CTA tiles, pairs of three widths and both arrangements with 256 x 256 outputs per CTA
    big = keys(8192, 8192, 8192)
    assert {(_native.VARIANT_CTA1, 256), (_native.VARIANT_CTA2, 256), (_native.VARIANT_CTA2, 192),
            (_native.VARIANT_CTA2, 512), (_native.VARIANT_CTA2_MCAST, 512)} <= big
    assert not any(v in (_native.VARIANT_SKINNY, _native.VARIANT_STREAMK) for v, _ in big)
    # a small square: no large tiles; the narrowest single-CTA tile joins when tiles are few
    small = keys(1024, 1024, 1024)
    assert (_native.VARIANT_CTA1, 64) in small and (_native.VARIANT_CTA2, 512) not in small
    # a decode batch: the short-A kernels (single CTAs and pairs) with the fitting and the next tile height, and
    # the 128-row kernels
    decode = keys(16, 14336, 4096)
    assert {(_native.VARIANT_SKINNY, 16), (_native.VARIANT_SKINNY, 32), (_native.VARIANT_SKINNY_PAIR, 16),
            (_native.VARIANT_CTA1, 128), (_native.VARIANT_STREAMK, 128)} <= decode
    assert {(_native.VARIANT_SKINNY, 128), (_native.VARIANT_SKINNY_PAIR, 128)} <= keys(100, 14336, 4096)
    assert (_native.VARIANT_SKINNY, 16) not in keys(40, 4096, 4096)
    # nothing to tune where only the CUDA-core kernel applies
    assert autotune.candidate_plans(512, 512, 100) == []


def test_plans_carry_the_store_path_the_shape_allows():
    assert all(p.tma_store == 1 for p in autotune.candidate_plans(2048, 2048, 2048))
    ragged = autotune.candidate_plans(2048, 2052, 2048)
    assert ragged and all(p.tma_store == 0 for p in ragged)
    # the large-tile kernels store by TMA only: not offered when N is not a multiple of 8
    assert not any(p.bn == 512 for p in autotune.candidate_plans(4096, 4100, 4096))


def test_header_records_options_but_no_paths():
    args = ["--squares", "256:8192:256", "--out", "somewhere/plan_table.txt", "--rounds", "3", "--log=x.jsonl", "--sustained"]
    assert autotune._options_without_paths(args) == ["--squares", "256:8192:256", "--rounds", "3", "--sustained"]


def test_refinements_vary_one_knob_at_a_time():
    """Second pass: band height and ring depth for whole tiles, k-ranges for stream-k, tile width and k-ranges for short A."""
    base = autotune.make_plan(_native.VARIANT_CTA2, 256, 8192)
    around = autotune.refinements(base, 8192, 8192, 8192)
    assert {p.group_m for p in around if p.stages == 0} >= {4, 8, 16}
    assert {p.stages for p in around if p.group_m == 0} == {4, 5}
    assert all((p.variant, p.bn) == (_native.VARIANT_CTA2, 256) for p in around)
    sk = autotune.refinements(autotune.make_plan(_native.VARIANT_STREAMK, 128, 4096), 96, 4096, 14336)
    assert {p.parts for p in sk} == {74, 148, 296}
    short = autotune.refinements(autotune.make_plan(_native.VARIANT_SKINNY, 16, 14336), 16, 14336, 4096)
    assert {p.group_m for p in short if p.parts == 0} >= {128, 104, 64} and {p.parts for p in short if p.group_m == 0} >= {1, 2, 4}
    # every refinement is a plan the library accepts
    import ctypes
    lib = _native.load()
    for p in around + sk + short:
        assert lib.b200_hgemm_plan_supported(8192, 8192, 8192, ctypes.byref(p)) == _native.OK or p.variant in (
            _native.VARIANT_SKINNY, _native.VARIANT_SKINNY_PAIR)


def test_plan_spelling_of_the_timing_tools():
    """abtest / timeline / profile_target spell a plan `variant:bn[:gN][:pN][:sN][:cN][:nt]`."""
    from cuda_hgemm_b200.abtest import parse_plan

    p = parse_plan("skinny:128:p4:c1")
    assert (p.variant, p.bn, p.parts, p.grid, p.group_m, p.tma_store) == (_native.VARIANT_SKINNY, 128, 4, 1, 0, 1)
    p = parse_plan("skinny2:64:g104:c2:nt")
    assert (p.variant, p.bn, p.group_m, p.grid, p.tma_store) == (_native.VARIANT_SKINNY_PAIR, 64, 104, 2, 0)
    p = parse_plan("cta2:288")
    assert (p.variant, p.bn, p.stages) == (_native.VARIANT_CTA2, 288, 0)
    assert parse_plan("cta2:256:s5").stages == 5
    # the wide pair tiles are among the candidates of a square
    assert {(_native.VARIANT_CTA2, 288), (_native.VARIANT_CTA2, 320)} <= keys(2304, 2304, 2304)
