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
    # a decode batch: the short-A kernel with the fitting and the largest tile height, and the 128-row kernels
    decode = keys(16, 14336, 4096)
    assert {(_native.VARIANT_SKINNY, 16), (_native.VARIANT_SKINNY, 64), (_native.VARIANT_CTA1, 128),
            (_native.VARIANT_STREAMK, 128)} <= decode
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
