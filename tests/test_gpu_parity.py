"""Parity of the CUDA kernels with the CPU oracle, through the C ABI, on a B200.

Tolerance (stated by the task this library is built to): max-norm relative error <= 1e-2 on the
FP16 output against the FP32-accumulate product of the same seeded inputs; ``assert_close_to_oracle``
additionally holds the kernels to 2e-3, what FP32 accumulation with one rounding should reach.
"""
import ctypes

import numpy as np
import pytest

from cuda_hgemm_b200 import _native, api
from oracle import hgemm_oracle as oracle
from tests.helpers import assert_close_to_oracle, make_inputs

pytestmark = pytest.mark.gpu

POISON = 0x7E00  # FP16 NaN: an element the kernel never wrote stays non-finite


def to_dev(x, device):
    import torch

    return torch.from_numpy(x).to(device)


def poisoned(M, N, device, extra_rows=0):
    import torch

    c = torch.full(((M + extra_rows) * N,), POISON, dtype=torch.int16, device=device).view(torch.float16)
    return c


def run(fn, A, B, device, plan=None):
    """Runs one entry point on poisoned C with canary rows behind it; returns C as numpy."""
    import torch

    M, K = A.shape
    N = B.shape[0]
    dA, dB = to_dev(A, device), to_dev(B, device)
    flat = poisoned(M, N, device, extra_rows=4)
    C = flat[: M * N].view(M, N)
    if plan is not None:
        api.hgemm_ex(dA, dB, C, plan)
    else:
        fn(dA, dB, C)
    torch.cuda.synchronize(device)
    assert api.last_device_error() == 0
    canary = flat[M * N:].view(torch.int16).cpu().numpy()
    assert (canary == POISON).all(), "kernel wrote past the end of C"
    return C.cpu().numpy()


def plan_of(variant, bn, parts=0, tma_store=1, group_m=0, grid=0):
    p = _native.Plan()
    p.variant, p.bn, p.parts, p.tma_store, p.group_m, p.grid = variant, bn, parts, tma_store, group_m, grid
    return p


SMALL_SHAPES = [
    (128, 256, 64),     # one tile, one k-block
    (128, 256, 256),    # one tile, ring of 4 stages exactly once
    (256, 256, 256),    # configuration 1 of the benchmark
    (384, 512, 320),    # 5 k-blocks: not a multiple of any stage count
    (512, 2048, 1024),  # the reference driver's default shape (reference src/main.cu:35-37)
    (200, 264, 136),    # tails in M, N and K
    (8, 8, 8),          # smaller than every tile dimension
    (1024, 1024, 1024),
]


@pytest.mark.parametrize("shape", SMALL_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_auto_dispatch_matches_oracle(cuda_device, shape):
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=2023)
    C = run(api.b200Hgemm, A, B, cuda_device)
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"auto {shape}")


def _seeded_shapes(count, seed):
    """Shapes drawn so that every branch of the dispatch is hit: decode batches, one to a few waves of
    tiles, ragged waves, K with and without a multiple of 8, N with and without."""
    rng = np.random.default_rng(seed)
    shapes = []
    for i in range(count):
        kind = i % 5
        if kind == 0:    # short A
            M = int(rng.integers(1, 65)); N = int(rng.integers(1, 40)) * 64 + int(rng.integers(0, 3)) * 4; K = int(rng.integers(1, 60)) * 64
        elif kind == 1:  # 65..128 rows
            M = int(rng.integers(65, 129)); N = int(rng.integers(2, 30)) * 128; K = int(rng.integers(2, 40)) * 64 + 8 * int(rng.integers(0, 8))
        elif kind == 2:  # a few tiles, tails everywhere
            M = int(rng.integers(129, 1500)); N = int(rng.integers(1, 190)) * 8; K = int(rng.integers(1, 190)) * 8
        elif kind == 3:  # around one to three waves of 128 x 256 tiles
            M = int(rng.integers(8, 24)) * 128; N = int(rng.integers(4, 12)) * 256; K = int(rng.integers(1, 9)) * 64
        else:            # anything, K not a multiple of 8 now and then
            M = int(rng.integers(1, 700)); N = int(rng.integers(1, 700)); K = int(rng.integers(1, 700))
        shapes.append((M, N, K))
    return shapes


@pytest.mark.parametrize("shape", _seeded_shapes(40, seed=20231), ids=lambda s: "x".join(map(str, s)))
def test_seeded_shapes_through_the_dispatch(cuda_device, shape):
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=M * 7 + N * 3 + K, dist="normal" if M <= 128 else "uniform")
    C = run(api.b200Hgemm, A, B, cuda_device)
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"auto {shape} plan {api.select_plan(M, N, K).as_dict()}")


@pytest.mark.parametrize("tma_store", [0, 1])
@pytest.mark.parametrize("bn", [64, 128, 192, 256])
@pytest.mark.parametrize("shape", [(128, 256, 64), (384, 512, 320), (200, 264, 136), (1024, 1536, 512)],
                         ids=lambda s: "x".join(map(str, s)))
def test_single_cta_tiles(cuda_device, shape, bn, tma_store):
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=1)
    C = run(None, A, B, cuda_device, plan_of(_native.VARIANT_CTA1, bn, tma_store=tma_store))
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"cta1 bn={bn} tma_store={tma_store} {shape}")


@pytest.mark.parametrize("bn", [128, 160, 192, 224, 256, 288, 320])  # 288 and 320: two MMAs side by side per tile
@pytest.mark.parametrize("shape", [(256, 256, 64), (256, 512, 320), (512, 2048, 1024), (328, 264, 136), (2048, 2048, 512),
                                   (3840, 3840, 192),   # 225 tiles of 256 x 256 on 74 pairs: several tiles per pair
                                   (1300, 3320, 136)],  # 78 such tiles, ragged in M, N and K
                         ids=lambda s: "x".join(map(str, s)))
def test_cta_pair_tiles(cuda_device, shape, bn):
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=2)
    C = run(None, A, B, cuda_device, plan_of(_native.VARIANT_CTA2, bn))
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"cta2 bn={bn} {shape}")


@pytest.fixture
def multicast_on():
    """Switches the single-GPU multicast kernels on for one test (they are off by default)."""
    from cuda_hgemm_b200 import build

    if not build.MULTICAST_SO.exists():
        pytest.skip("libb200_hgemm_mc.so is not part of this run (it is left out on multi-GPU runs)")
    if not api.enable_multicast(True):
        pytest.skip("this process may not use the multicast kernels (it drives several GPUs)")
    yield
    api.enable_multicast(False)


@pytest.mark.parametrize("shape", [(256, 512, 64), (256, 256, 320), (328, 776, 136), (1024, 2048, 1024), (2304, 2560, 512)],
                         ids=lambda s: "x".join(map(str, s)))
def test_cluster_multicast_pairs(cuda_device, multicast_on, shape):
    """The single-GPU companion kernel: CTA pairs in clusters of four, A slabs delivered by TMA multicast."""
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=12)
    C = run(None, A, B, cuda_device, plan_of(_native.VARIANT_CTA2_MCAST, 256))
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"multicast pairs {shape}")
    # same products in the same order as the plain pair kernel: bit-identical results
    C2 = run(None, A, B, cuda_device, plan_of(_native.VARIANT_CTA2, 256))
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))


@pytest.mark.parametrize("variant,bn,stages", [
    (_native.VARIANT_CTA1, 256, 3), (_native.VARIANT_CTA1, 128, 2), (_native.VARIANT_CTA1, 64, 3),
    (_native.VARIANT_CTA2, 256, 4), (_native.VARIANT_CTA2, 256, 5), (_native.VARIANT_CTA2, 128, 3),
], ids=lambda v: str(v))
def test_shallower_operand_rings(cuda_device, variant, bn, stages):
    """plan.stages: the whole-tile kernels with a ring one or two stages short of their default; same bits."""
    import torch

    M, N, K = 600, 776, 1096   # 18 k-blocks: several trips round every ring; tails in M, N and K
    A, B = make_inputs(M, N, K, seed=14)
    plan = plan_of(variant, bn)
    plan.stages = stages
    C = run(None, A, B, cuda_device, plan)
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"variant {variant} bn {bn} stages {stages}")
    assert np.array_equal(C.view(np.uint16), run(None, A, B, cuda_device, plan_of(variant, bn)).view(np.uint16))
    lib = _native.load()
    bad = plan_of(variant, bn)
    bad.stages = 9
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    dC = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
    assert lib.b200_hgemm_ex(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, N, K, ctypes.byref(bad), None) == _native.ERR_UNSUPPORTED


BIG_TILE_SHAPES = [
    (512, 256, 64),      # one pair tile, one k-block
    (512, 512, 256),     # one tile for a group of four, the ring of 4 stages exactly once
    (256, 256, 320),     # smaller than the tile: the second CTA of the pair works on padding
    (600, 776, 136),     # tails in M, N and K
    (1024, 2048, 1024),
    (2560, 2304, 512),   # several tiles per worker: tensor memory handed back and forth
    (6144, 5120, 576),   # more tiles than workers on every arrangement
    (520, 264, 8200),    # long k, 129 k-blocks
    (1300, 6656, 200),   # 78 pair tiles: one full wave of 74, the other four as eight 256 x 256 halves behind it; ragged M
    (2048, 16384, 320),  # one of eight row slabs of 16384^2: three full waves and 34 tiles as 68 halves
]


@pytest.mark.parametrize("shape", BIG_TILE_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_pair_tiles_of_256_rows_per_cta(cuda_device, shape):
    """512 x 256 pair tiles: two accumulators per CTA fill tensor memory, drain-first epilogue."""
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=21)
    C = run(None, A, B, cuda_device, plan_of(_native.VARIANT_CTA2, 512))
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"cta2 512x256 {shape}")
    # same products in the same order as the 256 x 256 pair kernel: bit-identical results
    C2 = run(None, A, B, cuda_device, plan_of(_native.VARIANT_CTA2, 256))
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))


@pytest.mark.parametrize("shape", BIG_TILE_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_cluster_multicast_groups_of_256_rows_per_cta(cuda_device, multicast_on, shape):
    """512 x 512 tiles on groups of four CTAs, A slab halves delivered by TMA multicast."""
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=22)
    C = run(None, A, B, cuda_device, plan_of(_native.VARIANT_CTA2_MCAST, 512))
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"multicast 512x512 {shape}")
    C2 = run(None, A, B, cuda_device, plan_of(_native.VARIANT_CTA2, 512))
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))


def test_multicast_kernels_are_off_until_asked_for_and_take_local_device_memory_only(cuda_device):
    """Default: the dispatch never picks them and an explicit plan is refused. Switched on: operands that
    are not allocations of the current GPU (here: pinned host memory) are refused before anything is launched."""
    import torch

    from cuda_hgemm_b200 import build

    lib = _native.load()
    if lib.b200_hgemm_multicast_state() == _native.MULTICAST_ON:
        api.enable_multicast(False)
    M = N = K = 512
    A, B = make_inputs(M, N, K, seed=24)
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    C = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
    for bn in (256, 512):
        with pytest.raises(_native.HgemmError) as e:
            api.hgemm_ex(dA, dB, C, plan_of(_native.VARIANT_CTA2_MCAST, bn))
        assert e.value.status == _native.ERR_UNSUPPORTED
    assert api.select_plan_untuned(16384, 16384, 16384).variant == _native.VARIANT_CTA2
    if not build.MULTICAST_SO.exists() or not api.enable_multicast(True):
        return
    try:
        hA = torch.from_numpy(A).pin_memory()
        rc = lib.b200_hgemm_ex(hA.data_ptr(), dB.data_ptr(), C.data_ptr(), M, N, K,
                               ctypes.byref(plan_of(_native.VARIANT_CTA2_MCAST, 512)), None)
        assert rc == _native.ERR_UNSUPPORTED
        api.hgemm_ex(dA, dB, C, plan_of(_native.VARIANT_CTA2_MCAST, 512))
        torch.cuda.synchronize()
        assert_close_to_oracle(C.cpu().numpy(), oracle.gemm_f32(A, B), "multicast after a refused call")
    finally:
        api.enable_multicast(False)


def test_large_tiles_refuse_what_their_epilogue_cannot_store(cuda_device):
    """Their epilogue is TMA stores only: N must be a multiple of 8 halves and the plan must say TMA."""
    import torch

    A, B = make_inputs(512, 1001, 512, seed=23)
    dA, dB = (torch.from_numpy(x).to(cuda_device) for x in (A, B))
    C = torch.empty((512, 1001), dtype=torch.float16, device=cuda_device)
    for variant in (_native.VARIANT_CTA2, _native.VARIANT_CTA2_MCAST):
        with pytest.raises(_native.HgemmError) as e:
            api.hgemm_ex(dA, dB, C, plan_of(variant, 512))
        assert e.value.status == _native.ERR_UNSUPPORTED
    A2, B2 = make_inputs(512, 1024, 512, seed=23)
    dA2, dB2 = (torch.from_numpy(x).to(cuda_device) for x in (A2, B2))
    C2 = torch.empty((512, 1024), dtype=torch.float16, device=cuda_device)
    with pytest.raises(_native.HgemmError) as e:
        api.hgemm_ex(dA2, dB2, C2, plan_of(_native.VARIANT_CTA2, 512, tma_store=0))
    assert e.value.status == _native.ERR_UNSUPPORTED


@pytest.mark.parametrize("K", [1096, 1160])  # 18 k-blocks; 19, so that the last pair of k-blocks is half past K
@pytest.mark.parametrize("parts", [0, 1, 7, 33, 148, 400])
@pytest.mark.parametrize("bn", [64, 128, 256])
def test_stream_k_ranges(cuda_device, bn, parts, K):
    M, N = 200, 1032  # tails everywhere
    A, B = make_inputs(M, N, K, seed=3)
    C = run(None, A, B, cuda_device, plan_of(_native.VARIANT_STREAMK, bn, parts=parts))
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"stream-k bn={bn} parts={parts}")


SHORT_A_CASES = [
    # M, N, K, rows of A per tile, k-ranges per column tile (0 = the library's choice)
    (16, 128, 64, 16, 0),      # one tile, one k-block: half a stage
    (16, 256, 128, 16, 0),     # exactly one stage of two k-blocks
    (1, 128, 192, 16, 0),      # a single row; three k-blocks
    (9, 520, 200, 16, 0),      # tails in M, N (not a multiple of 8) and K
    (16, 1024, 4096, 16, 0),
    (16, 4096, 3584, 16, 3),   # three k-ranges of 19, 19 and 18 k-blocks
    (17, 264, 136, 32, 2),
    (32, 1000, 1096, 32, 0),
    (33, 1024, 3584, 64, 0),
    (64, 777, 320, 64, 5),     # as many k-ranges as k-blocks
    (64, 3584, 1024, 64, 0),
]


@pytest.mark.parametrize("case", SHORT_A_CASES, ids=lambda c: "x".join(map(str, c[:3])) + f"-mt{c[3]}-p{c[4]}")
def test_short_a_kernel(cuda_device, case):
    """M <= 64: B on the MMA's row operand, C accumulated transposed, k-ranges summed from FP32 partials."""
    M, N, K, mt, parts = case
    A, B = make_inputs(M, N, K, seed=31, dist="normal")
    C = run(None, A, B, cuda_device, plan_of(_native.VARIANT_SKINNY, mt, parts=parts))
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"short-A mt={mt} parts={parts} {(M, N, K)}")
    # the same plan twice gives the same bits (the k-ranges are summed in a fixed order)
    C2 = run(None, A, B, cuda_device, plan_of(_native.VARIANT_SKINNY, mt, parts=parts))
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))
    # and so do CTA pairs: the same products in the same order
    C3 = run(None, A, B, cuda_device, plan_of(_native.VARIANT_SKINNY_PAIR, mt, parts=parts))
    assert np.array_equal(C.view(np.uint16), C3.view(np.uint16))
    # plain stores instead of the staged TMA store
    C4 = run(None, A, B, cuda_device, plan_of(_native.VARIANT_SKINNY, mt, parts=parts, tma_store=0))
    assert np.array_equal(C.view(np.uint16), C4.view(np.uint16))


SHORT_A_WIDTH_CASES = [
    # M, N, K, rows of A per tile, columns of C per tile (0 = the library's choice), k-ranges
    (16, 1040, 512, 16, 104, 0),     # ten tiles of 104 columns
    (16, 1000, 200, 16, 72, 0),      # N not a multiple of the width nor of 8; tails in K
    (64, 14336, 256, 64, 0, 0),      # the library's own choice for the decode shape: 138 tiles of 104
    (48, 2048, 1096, 64, 64, 3),     # narrow tiles and k-ranges together
    (128, 512, 256, 128, 0, 0),      # 128 rows of A per tile
    (100, 1032, 1096, 128, 0, 0),    # tails in M, N, K
    (128, 14336, 512, 128, 0, 0),    # 138 tiles of 104 columns
    (65, 4096, 3584, 128, 0, 0),     # few column tiles: k cut into ranges, FP32 partials summed
    (128, 777, 320, 128, 88, 5),
    (8, 136, 64, 16, 8, 0),          # the narrowest tile there is
]


@pytest.mark.parametrize("variant", [_native.VARIANT_SKINNY, _native.VARIANT_SKINNY_PAIR], ids=["single", "pairs"])
@pytest.mark.parametrize("case", SHORT_A_WIDTH_CASES, ids=lambda c: "x".join(map(str, c[:3])) + f"-mt{c[3]}-w{c[4]}-p{c[5]}")
def test_short_a_kernel_tile_widths_and_128_rows(cuda_device, case, variant):
    """Column tiles narrower than 128 (the TMA box of B has fewer rows than the MMA multiplies), up to 128 rows
    of A, single CTAs and CTA pairs that share the rows of A."""
    M, N, K, mt, width, parts = case
    A, B = make_inputs(M, N, K, seed=33, dist="normal")
    plan = plan_of(variant, mt, parts=parts, group_m=width)
    C = run(None, A, B, cuda_device, plan)
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"short-A mt={mt} width={width} parts={parts} {(M, N, K)}")
    C2 = run(None, A, B, cuda_device, plan)
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))


CLUSTER_SUM_CASES = [
    # M, N, K, rows of A per tile, columns of C per tile (0 = the library's choice), k-ranges
    (16, 256, 256, 16, 0, 2),        # two k-ranges of two k-blocks; each owner sums 8 rows
    (1, 128, 192, 16, 0, 3),         # one row: owners 1 and 2 have nothing to sum
    (9, 520, 200, 16, 0, 4),         # tails in M, N (not a multiple of 8) and K; rows 3 + 3 + 3 + 0
    (16, 4096, 3584, 16, 0, 4),
    (17, 264, 136, 32, 0, 2),
    (32, 1000, 1096, 32, 72, 8),     # the largest cluster of single CTAs, narrow tiles
    (64, 4096, 3584, 64, 0, 0),      # the library's choice: 32 tiles, four k-ranges
    (100, 1032, 1096, 128, 0, 3),    # 34 + 34 + 32 rows
    (128, 4096, 3584, 128, 0, 4),    # the transposed decode shape with a shorter K
    (128, 777, 320, 128, 88, 5),     # five k-ranges of one k-block: pairs would need a cluster of ten
]


@pytest.mark.parametrize("variant", [_native.VARIANT_SKINNY, _native.VARIANT_SKINNY_PAIR], ids=["single", "pairs"])
@pytest.mark.parametrize("case", CLUSTER_SUM_CASES, ids=lambda c: "x".join(map(str, c[:3])) + f"-mt{c[3]}-w{c[4]}-p{c[5]}")
def test_short_a_kernel_sums_k_ranges_inside_clusters(cuda_device, case, variant):
    """plan.grid = 1: the k-ranges of a column tile are one thread-block cluster and add their partial results through
    distributed shared memory; plan.grid = 2: through the FP32 workspace and the summing kernel. Same products, same
    order of addition: the same bits. A cluster larger than eight CTAs is refused."""
    M, N, K, mt, width, parts = case
    A, B = make_inputs(M, N, K, seed=35, dist="normal")
    cg = 2 if variant == _native.VARIANT_SKINNY_PAIR else 1
    on_chip = plan_of(variant, mt, parts=parts, group_m=width, grid=1)
    if parts * cg > 8:
        import torch

        dA, dB = (torch.from_numpy(x).to(cuda_device) for x in (A, B))
        C = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
        with pytest.raises(_native.HgemmError) as e:
            api.hgemm_ex(dA, dB, C, on_chip)
        assert e.value.status == _native.ERR_UNSUPPORTED
        return
    assert api.workspace_bytes(M, N, K, on_chip) == 0
    C = run(None, A, B, cuda_device, on_chip)
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"short-A cluster sum mt={mt} width={width} parts={parts} {(M, N, K)}")
    through_workspace = plan_of(variant, mt, parts=parts, group_m=width, grid=2)
    assert api.workspace_bytes(M, N, K, through_workspace) > 0
    C2 = run(None, A, B, cuda_device, through_workspace)
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))
    C3 = run(None, A, B, cuda_device, on_chip)
    assert np.array_equal(C.view(np.uint16), C3.view(np.uint16))


def test_short_a_kernel_falls_back_to_the_workspace_when_the_clusters_do_not_fit(cuda_device):
    """The library's own choice of summing inside clusters needs all clusters on the device at once; where the device
    (here: a pretended one) holds fewer, the same k-ranges go through the workspace: two launches instead of one, the
    same bits. A plan that asks for the clusters still gets them."""
    M, N, K = 16, 4096, 3584
    A, B = make_inputs(M, N, K, seed=37, dist="normal")
    auto = plan_of(_native.VARIANT_SKINNY, 16)       # 32 tiles, four k-ranges: 32 clusters of four
    lib = _native.load()
    before = api.launch_count()
    C = run(None, A, B, cuda_device, auto)
    assert api.launch_count() - before == 1
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), "short-A, clusters")
    lib.b200_debug_cluster_capacity(8)
    try:
        before = api.launch_count()
        C2 = run(None, A, B, cuda_device, auto)
        assert api.launch_count() - before == 2      # the GEMM and the summing kernel
        before = api.launch_count()
        C3 = run(None, A, B, cuda_device, plan_of(_native.VARIANT_SKINNY, 16, grid=1))
        assert api.launch_count() - before == 1
    finally:
        lib.b200_debug_cluster_capacity(0)
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))
    assert np.array_equal(C.view(np.uint16), C3.view(np.uint16))


def test_short_a_kernel_refuses_more_rows_than_its_tile(cuda_device):
    import torch

    A, B = make_inputs(40, 256, 256, seed=32)
    dA, dB = (torch.from_numpy(x).to(cuda_device) for x in (A, B))
    C = torch.empty((40, 256), dtype=torch.float16, device=cuda_device)
    with pytest.raises(_native.HgemmError) as e:
        api.hgemm_ex(dA, dB, C, plan_of(_native.VARIANT_SKINNY, 32))
    assert e.value.status == _native.ERR_UNSUPPORTED
    with pytest.raises(_native.HgemmError) as e:
        api.hgemm_ex(dA, dB, C, plan_of(_native.VARIANT_SKINNY, 48))
    assert e.value.status == _native.ERR_UNSUPPORTED


HYBRID_CASES = [
    # M, N, K, bn, parts (0 = one per SM)
    (2304, 2304, 512, 256, 0),    # 162 tiles: one full wave whole, 14 tiles cut into k-ranges
    (2304, 2304, 512, 128, 0),    # 324 tiles, two whole per worker, 28 cut; two k-blocks per stage
    (1000, 1032, 1096, 256, 7),   # tails everywhere; 40 tiles on 7 workers: 35 whole, 5 cut
    (1000, 1032, 1096, 64, 7),
    (200, 1032, 1096, 128, 33),   # fewer tiles than workers: nothing whole, plain stream-k
    (1280, 2560, 320, 256, 10),   # 100 tiles on 10 workers: nothing left to cut
    (3840, 3840, 256, 256, 148),  # 6 cut tiles of 4 k-blocks: fewer units than workers
]


@pytest.mark.parametrize("case", HYBRID_CASES, ids=lambda c: "x".join(map(str, c[:3])) + f"-bn{c[3]}-p{c[4]}")
def test_whole_tiles_then_k_ranges(cuda_device, case):
    """HYBRID: full waves of tiles computed whole, the ragged rest cut into k-ranges and summed."""
    M, N, K, bn, parts = case
    A, B = make_inputs(M, N, K, seed=41)
    C = run(None, A, B, cuda_device, plan_of(_native.VARIANT_HYBRID, bn, parts=parts, tma_store=1 if N % 8 == 0 else 0))
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"hybrid bn={bn} parts={parts} {(M, N, K)}")
    # poison the workspace's idea of "clean": a second run must not depend on what the first left behind
    C2 = run(None, A, B, cuda_device, plan_of(_native.VARIANT_HYBRID, bn, parts=parts, tma_store=1 if N % 8 == 0 else 0))
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))


HYBRID_PAIR_CASES = [
    # M, N, K, bn, parts (0 = one per two SMs)
    (2304, 2304, 512, 256, 0),    # 81 pair tiles: 74 whole, 7 cut into k-ranges over all pairs
    (2304, 2304, 512, 128, 0),    # 162 tiles of 256 x 128: two whole per pair, 14 cut; two k-blocks per stage
    (1792, 1792, 1096, 256, 0),   # 49 tiles on 74 pairs: nothing whole, every tile cut
    (1000, 1032, 1096, 256, 7),   # tails everywhere; 20 tiles on 7 pairs: 14 whole, 6 cut
    (1000, 1032, 1096, 128, 5),
    (300, 520, 8200, 256, 33),    # fewer tiles than pairs, long k
    (1280, 2560, 320, 256, 10),   # 50 tiles on 10 pairs: nothing left to cut
    (3840, 3840, 256, 256, 74),   # 3 cut tiles of 4 k-blocks: fewer units than pairs
]


@pytest.mark.parametrize("case", HYBRID_PAIR_CASES, ids=lambda c: "x".join(map(str, c[:3])) + f"-bn{c[3]}-p{c[4]}")
def test_whole_pair_tiles_then_k_ranges(cuda_device, case):
    """HYBRID_PAIR: full waves of 256-row pair tiles computed whole, the ragged rest cut into k-ranges and summed."""
    M, N, K, bn, parts = case
    A, B = make_inputs(M, N, K, seed=43)
    plan = plan_of(_native.VARIANT_HYBRID_PAIR, bn, parts=parts, tma_store=1 if N % 8 == 0 else 0)
    C = run(None, A, B, cuda_device, plan)
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"hybrid pairs bn={bn} parts={parts} {(M, N, K)}")
    C2 = run(None, A, B, cuda_device, plan)
    assert np.array_equal(C.view(np.uint16), C2.view(np.uint16))


@pytest.mark.parametrize("M", [16, 32, 64, 128])
def test_skinny_decode_shapes(cuda_device, M):
    # decode-like: activations ~ N(0,1), weights ~ N(0, 1/K); N and K scaled down 4x from 14336 x 4096
    for N, K in ((3584, 1024), (1024, 3584)):
        A, B = make_inputs(M, N, K, seed=4, dist="normal")
        ref = oracle.gemm_f32(A, B)
        for fn in (api.b200Hgemm, api.b200HgemmStreamK, api.b200HgemmSplitK):
            C = run(fn, A, B, cuda_device)
            assert_close_to_oracle(C, ref, f"{fn.__name__} {M}x{N}x{K}")


def test_fixed_variant_entry_points(cuda_device):
    M, N, K = 512, 768, 512
    A, B = make_inputs(M, N, K, seed=5)
    ref = oracle.gemm_f32(A, B)
    for fn in (api.b200Hgemm, api.b200HgemmCta1, api.b200HgemmCta2, api.b200HgemmSplitK, api.b200HgemmStreamK,
               api.b200HgemmSimt):
        assert_close_to_oracle(run(fn, A, B, cuda_device), ref, fn.__name__)


def test_any_shape_goes_through_the_cuda_core_kernel(cuda_device):
    # K % 8 != 0: no TMA row pitch; the library still computes on the GPU
    g = np.load(str(__import__("pathlib").Path(__file__).parent / "golden" / "odd_k_48x40x100.npz"))
    C = run(api.b200Hgemm, g["A"], g["B"], cuda_device)
    assert_close_to_oracle(C, g["ref_f32"], "odd K")


def test_golden_fixtures_on_device(cuda_device):
    from pathlib import Path

    for path in sorted((Path(__file__).parent / "golden").glob("*.npz")):
        g = np.load(path)
        C = run(api.b200Hgemm, g["A"], g["B"], cuda_device)
        assert_close_to_oracle(C, g["ref_f32"], path.stem)
        # against the float64 product rounded to FP16: at most one FP16 step of each value
        g16 = g["ref_f16"].astype(np.float64)
        step = 2.0 ** -10 * np.abs(g16) + 1e-4 * np.abs(g16).max()
        assert (np.abs(C.astype(np.float64) - g16) <= step).all(), path.stem


def test_results_are_reproducible_bit_for_bit(cuda_device):
    M, N, K = 256, 1024, 2048
    A, B = make_inputs(M, N, K, seed=6)
    for plan in (plan_of(_native.VARIANT_CTA1, 256), plan_of(_native.VARIANT_CTA2, 256),
                 plan_of(_native.VARIANT_STREAMK, 128), plan_of(_native.VARIANT_STREAMK, 64, parts=97)):
        first = run(None, A, B, cuda_device, plan).view(np.uint16)
        for _ in range(3):
            again = run(None, A, B, cuda_device, plan).view(np.uint16)
            assert np.array_equal(first, again), f"variant {plan.variant} is not deterministic"


def test_row_slabs_equal_rows_of_the_full_product(cuda_device):
    # the multi-GPU partition: each slab is computed by the same tile code as the full problem
    from cuda_hgemm_b200.partition import row_slabs

    M, N, K = 2048, 1024, 512
    A, B = make_inputs(M, N, K, seed=8)
    plan = plan_of(_native.VARIANT_CTA1, 256)
    full = run(None, A, B, cuda_device, plan).view(np.uint16)
    for lo, hi in row_slabs(M, 4):
        slab = run(None, A[lo:hi], B, cuda_device, plan).view(np.uint16)
        assert np.array_equal(slab, full[lo:hi])


def test_linearity_at_full_size(cuda_device):
    """Size-independent property at a benchmark-size shape: (A1 + A2) * B = A1*B + A2*B when the
    sums are exact in FP16 (small integers), checked on all of C; plus sampled rows vs the oracle."""
    import torch

    M = N = K = 4096
    rng = np.random.default_rng(9)
    A1 = rng.integers(-2, 3, size=(M, K)).astype(np.float16)
    A2 = rng.integers(-2, 3, size=(M, K)).astype(np.float16)
    B = (rng.integers(-2, 3, size=(N, K)) / 64.0).astype(np.float16)
    dB = to_dev(B, cuda_device)
    outs = []
    for a in (A1, A2, A1 + A2):
        C = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
        api.b200Hgemm(to_dev(a, cuda_device), dB, C)
        outs.append(C)
    torch.cuda.synchronize()
    assert api.last_device_error() == 0
    # every partial sum is a multiple of 1/64 below 2^11/64: exact in FP32, and the outputs are exact
    # in FP16 whenever |C| < 32, so linearity must hold bit for bit there
    c1, c2, c12 = (o.float() for o in outs)
    exact = (c1.abs() < 16) & (c2.abs() < 16)
    assert torch.equal((c1 + c2)[exact], c12[exact])
    rows = [0, 127, 128, 2049, M - 1]
    ref = np.stack([oracle.gemm_f32_rows(A1 + A2, B, r, 1)[0] for r in rows])
    assert_close_to_oracle(outs[2][rows].cpu().numpy(), ref, "4096^3 sampled rows")


def test_large_square_sampled_rows(cuda_device):
    import torch

    M = N = K = 8192
    A, B = make_inputs(M, N, K, seed=10)
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    C = poisoned(M, N, cuda_device).view(M, N)
    api.b200Hgemm(dA, dB, C)
    torch.cuda.synchronize()
    assert api.last_device_error() == 0
    assert torch.isfinite(C).all()
    # the first and last row block and one in the middle cover every column tile and k-block
    for row0 in (0, 4096 + 128, M - 128):
        ref = oracle.gemm_f32_rows(A, B, row0, 128)
        assert_close_to_oracle(C[row0:row0 + 128].cpu().numpy(), ref, f"8192^3 rows {row0}..")
    # the CTA-pair and single-CTA kernels agree on all of C to one FP16 step (same products, other order)
    C1 = torch.empty_like(C)
    api.b200HgemmCta1(dA, dB, C1)
    torch.cuda.synchronize()
    diff = (C.float() - C1.float()).abs()
    assert (diff <= 2.0 ** -9 * C1.float().abs() + 1e-3).all()


def test_host_pointer_entry_point(cuda_device):
    import torch

    for M, N, K in ((256, 256, 256), (2048, 512, 256), (300, 264, 136)):
        A, B = make_inputs(M, N, K, seed=11)
        hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
        hC = torch.full((M, N), float("nan"), dtype=torch.float16).pin_memory()
        api.hgemm_host(hA, hB, hC)
        assert_close_to_oracle(hC.numpy(), oracle.gemm_f32(A, B), f"host {M}x{N}x{K}")


def test_host_entry_point_with_b_resident_on_the_device(cuda_device):
    """b200_hgemm_host_a: A up and C down in slabs, B already on the GPU; same bits as the all-host entry point."""
    import torch

    for M, N, K in ((256, 256, 256), (4096, 512, 256), (2048 + 512, 264, 136), (300, 264, 136)):
        A, B = make_inputs(M, N, K, seed=13)
        hA = torch.from_numpy(A).pin_memory()
        hC = torch.full((M, N), float("nan"), dtype=torch.float16).pin_memory()
        hC2 = torch.full((M, N), float("nan"), dtype=torch.float16).pin_memory()
        dB = to_dev(B, cuda_device)
        api.hgemm_host_a(hA, dB, hC)
        assert_close_to_oracle(hC.numpy(), oracle.gemm_f32(A, B), f"host A, resident B {M}x{N}x{K}")
        api.hgemm_host(hA, torch.from_numpy(B).pin_memory(), hC2)
        assert np.array_equal(hC.numpy().view(np.uint16), hC2.numpy().view(np.uint16))


def test_host_entry_point_that_waits_for_b_on_events(cuda_device):
    """b200_hgemm_host_a_after: B is still being written on another stream when the call is made; the uploads of
    A wait for one event, the multiplies for the other."""
    import torch

    M, N, K = 2048 + 512, 520, 264
    A, B = make_inputs(M, N, K, seed=15)
    hA, hB = torch.from_numpy(A).pin_memory(), torch.from_numpy(B).pin_memory()
    hC = torch.full((M, N), float("nan"), dtype=torch.float16).pin_memory()
    dB = torch.zeros((N, K), dtype=torch.float16, device=cuda_device)
    side = torch.cuda.Stream(device=cuda_device)
    with torch.cuda.stream(side):
        started = torch.cuda.Event()
        started.record()
        torch.cuda._sleep(20_000_000)          # B arrives late: about 10 ms of spinning first
        dB.copy_(hB, non_blocking=True)
        complete = torch.cuda.Event()
        complete.record()
    api.hgemm_host_a(hA, dB, hC, upload_after=started, gemm_after=complete)
    assert_close_to_oracle(hC.numpy(), oracle.gemm_f32(A, B), "host A behind events")
    side.synchronize()


def _single_process_group_case(devices, M, N, K):
    import torch

    from cuda_hgemm_b200.multi_gpu import SingleProcessGroup

    A, B = make_inputs(M, N, K, seed=51)
    ref = oracle.gemm_f32(A, B)
    with SingleProcessGroup(devices) as group:
        slabs = [group.slab(M, i) for i in range(len(devices))]
        assert slabs[0][0] == 0 and slabs[-1][1] == M and all(a[1] == b[0] for a, b in zip(slabs, slabs[1:]))
        dA = [torch.from_numpy(A[lo:hi]).to(f"cuda:{d}") for d, (lo, hi) in zip(devices, slabs)]
        dB = [torch.from_numpy(B).to(f"cuda:{d}") for d in devices]
        dC = [torch.full((hi - lo, N), float("nan"), dtype=torch.float16, device=f"cuda:{d}") for d, (lo, hi) in zip(devices, slabs)]
        full = [torch.full((M, N), float("nan"), dtype=torch.float16, device=f"cuda:{d}") for d in devices]
        for _ in range(2):  # the second call reuses streams, events and cached tensor maps
            group.hgemm(dA, dB, dC, M)
            group.gather_c(dC, full, M, N)
            group.synchronize()
        assert group.elapsed_ms_max() > 0.0
        for d in devices:
            with torch.cuda.device(d):
                assert api.last_device_error() == 0
        for (lo, hi), c in zip(slabs, dC):
            if hi > lo:
                assert_close_to_oracle(c.cpu().numpy(), ref[lo:hi], f"slab rows {lo}:{hi}")
        # the gathered copies are the slabs, bit for bit, on every device
        whole = np.concatenate([c.cpu().numpy() for c in dC if c.shape[0]], axis=0)
        for f in full:
            assert np.array_equal(f.cpu().numpy().view(np.uint16), whole.view(np.uint16))
        # and a slab is what the single-GPU call computes for those rows
        single = run(api.b200Hgemm, A[slabs[0][0]:slabs[0][1]], B, torch.device(f"cuda:{devices[0]}"))
        assert np.array_equal(single.view(np.uint16), dC[0].cpu().numpy().view(np.uint16))


def test_single_process_group_on_one_device(cuda_device):
    """The b200_mg_* entry points with a group of one: the same code path as with eight."""
    _single_process_group_case([0], 640, 520, 328)


def test_single_process_group_on_all_devices(cuda_device):
    import torch

    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("one GPU in this run")
    _single_process_group_case(list(range(n)), 128 * (2 * n + 1) + 40, 1032, 576)  # uneven slabs and a ragged last one


def test_single_process_group_rejects_bad_device_lists(cuda_device):
    import ctypes

    lib = _native.load()
    handle = ctypes.c_void_p()
    for devices in ([], [0, 0], [-1], [4096]):
        arr = (ctypes.c_int * max(1, len(devices)))(*devices)
        assert lib.b200_mg_create(arr, len(devices), ctypes.byref(handle)) == _native.ERR_INVALID_ARG


FUSED_CASES = [
    # M, N, K, alpha, beta, bias?, in place?
    (256, 256, 256, 0.5, 0.0, False, False),     # alpha only
    (384, 512, 320, 1.0, 0.0, True, False),      # bias only
    (200, 264, 136, -1.25, 0.75, True, False),   # everything, tails in M, N, K
    (200, 1001, 136, 2.0, -0.5, True, False),    # N not a multiple of 8: guarded loads and stores
    (1024, 1536, 512, 1.0, 1.0, False, True),    # C += A * B^T in place
    (2304, 2304, 256, 0.25, 2.0, True, True),    # pairs on 256 x 192
    (16, 1024, 2048, 1.5, 0.5, True, False),     # a decode batch: the short-A kernel
    (16, 4096, 14336, 1.0, 1.0, True, True),     # the short-A kernel with k cut into ranges: epilogue in the summing kernel
    (96, 4096, 1024, 1.0, 0.5, True, True),      # the short-A kernel on CTA pairs
    (100, 512, 4096, 0.5, 0.5, True, False),     # k-ranges over 128-row tiles
    (4096, 4096, 1536, 1.0, 0.5, True, False),   # many waves of pairs
    (4096, 4096, 4096, 1.0, -1.0, True, True),   # 256 x 256 outputs per CTA
]


@pytest.mark.parametrize("case", FUSED_CASES, ids=lambda c: "x".join(map(str, c[:3])) + f"-a{c[3]}-b{c[4]}")
def test_fused_epilogue(cuda_device, case):
    """C = alpha * A B^T + beta * c_in + bias in one kernel, against the same expression on the oracle's product."""
    import torch

    M, N, K, alpha, beta, with_bias, in_place = case
    A, B = make_inputs(M, N, K, seed=61)
    rng = np.random.default_rng(62)
    c_in = rng.uniform(-4, 4, size=(M, N)).astype(np.float16)
    bias = rng.uniform(-2, 2, size=(N,)).astype(np.float16)
    ref = alpha * oracle.gemm_f32(A, B)
    if beta != 0.0:
        ref = ref + np.float32(beta) * c_in.astype(np.float32)
    if with_bias:
        ref = ref + bias.astype(np.float32)[None, :]
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    d_bias = to_dev(bias, cuda_device) if with_bias else None
    if in_place:
        C = to_dev(c_in, cuda_device).clone()
        api.hgemm_fused(dA, dB, C, alpha, beta, d_bias, C)
    else:
        C = poisoned(M, N, cuda_device).view(M, N)
        api.hgemm_fused(dA, dB, C, alpha, beta, d_bias, to_dev(c_in, cuda_device) if beta != 0.0 else None)
    torch.cuda.synchronize(cuda_device)
    assert api.last_device_error() == 0
    assert_close_to_oracle(C.cpu().numpy(), ref.astype(np.float32), f"fused {case}")


@pytest.mark.parametrize("shape", [(512, 768, 448), (16, 2048, 1024), (128, 4096, 2048), (2560, 2304, 1536)],
                         ids=lambda s: "x".join(map(str, s)))
def test_fused_epilogue_with_identity_matches_the_plain_product(cuda_device, shape):
    """alpha = 1, beta = 0, no bias: the same kernel family as the plain entry point, the same bits."""
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=63)
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    C = poisoned(M, N, cuda_device).view(M, N)
    api.hgemm_fused(dA, dB, C, 1.0, 0.0)
    plain = run(api.b200Hgemm, A, B, cuda_device)
    assert np.array_equal(C.cpu().numpy().view(np.uint16), plain.view(np.uint16))


FUSED_PLAN_CASES = [
    # M, N, K, variant, bn, parts, tma_store
    (1024, 2048, 1024, _native.VARIANT_CTA2, 512, 0, 1),      # 256 x 256 outputs per CTA, several tiles per CTA
    (600, 776, 136, _native.VARIANT_CTA2, 512, 0, 1),         # the same with tails in M, N and K
    (1300, 6656, 200, _native.VARIANT_CTA2, 512, 0, 1),       # a full wave and a tail of half tiles on the other pair kernel
    (1300, 3320, 136, _native.VARIANT_CTA2, 256, 0, 1),       # more 256 x 256 tiles than pairs, ragged in M, N and K
    (384, 512, 320, _native.VARIANT_CTA1, 192, 0, 1),
    (600, 776, 520, _native.VARIANT_CTA2, 192, 0, 1),
    (600, 776, 520, _native.VARIANT_CTA2, 160, 0, 1),         # the tile's last 32 columns leave by plain stores
    (1300, 3320, 136, _native.VARIANT_CTA2, 224, 0, 1),
    (1300, 3320, 136, _native.VARIANT_CTA2, 288, 0, 1),       # wider than one MMA; one accumulator, several tiles per pair
    (600, 776, 520, _native.VARIANT_CTA2, 320, 0, 0),
    (200, 1032, 1096, _native.VARIANT_STREAMK, 128, 33, 1),   # whole and cut tiles in one launch
    (200, 1032, 1096, _native.VARIANT_STREAMK, 64, 7, 0),
    (1000, 1032, 1096, _native.VARIANT_HYBRID, 256, 7, 1),
    (16, 4096, 3584, _native.VARIANT_SKINNY, 16, 3, 1),
    (40, 1000, 520, _native.VARIANT_SKINNY, 64, 0, 1),        # N % 8 != 0: by element
    (128, 2048, 1024, _native.VARIANT_SKINNY_PAIR, 128, 0, 1),
    (65, 1032, 1096, _native.VARIANT_SKINNY_PAIR, 128, 2, 1),
    # the same two with the k-ranges summed through the workspace (an eighth field: plan.grid = 2) instead of on chip
    (16, 4096, 3584, _native.VARIANT_SKINNY, 16, 3, 1, 2),
    (65, 1032, 1096, _native.VARIANT_SKINNY_PAIR, 128, 2, 1, 2),
]


@pytest.mark.parametrize("c_dtype", ["float16", "bfloat16", "float32"])
@pytest.mark.parametrize("case", FUSED_PLAN_CASES, ids=lambda c: "x".join(map(str, c[:3])) + f"-v{c[3]}-bn{c[4]}-p{c[5]}" + ("-ws" if len(c) > 7 else ""))
def test_fused_epilogue_on_every_kernel_family_and_output_type(cuda_device, case, c_dtype):
    """alpha, beta * c_in and bias on an explicit plan, C (and c_in) as FP16, BF16 or FP32."""
    import torch

    M, N, K, variant, bn, parts, tma_store = case[:7]
    dtype = getattr(torch, c_dtype)
    A, B = make_inputs(M, N, K, seed=66)
    rng = np.random.default_rng(67)
    alpha, beta = 0.75, -0.5
    c_in = torch.from_numpy(rng.uniform(-4, 4, size=(M, N)).astype(np.float32)).to(dtype)
    bias = rng.uniform(-2, 2, size=(N,)).astype(np.float16)
    ref = (alpha * oracle.gemm_f32(A, B) + np.float32(beta) * c_in.float().numpy() + bias.astype(np.float32)[None, :])
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    C = torch.full((M, N), float("nan"), dtype=dtype, device=cuda_device)
    plan = plan_of(variant, bn, parts=parts, tma_store=tma_store if N % 8 == 0 else 0, grid=case[7] if len(case) > 7 else 0)
    if variant == _native.VARIANT_CTA2 and bn == 512 and c_dtype == "float32":
        with pytest.raises(_native.HgemmError) as e:
            api.hgemm_fused(dA, dB, C, alpha, beta, to_dev(bias, cuda_device), c_in.to(cuda_device), plan=plan)
        assert e.value.status == _native.ERR_UNSUPPORTED
        return
    api.hgemm_fused(dA, dB, C, alpha, beta, to_dev(bias, cuda_device), c_in.to(cuda_device), plan=plan)
    torch.cuda.synchronize(cuda_device)
    assert api.last_device_error() == 0
    got = C.float().cpu().numpy()
    assert np.isfinite(got).all()
    if c_dtype == "float16":
        assert_close_to_oracle(C.cpu().numpy(), ref.astype(np.float32), f"fused {case}")
        return
    # FP32 output keeps the accumulator: only the order of summation differs from the oracle's; BF16 rounds once to 8 bits
    tol = 2e-5 if c_dtype == "float32" else 2.0 ** -8
    err = np.abs(got - ref).max() / np.abs(ref).max()
    assert err <= tol, f"{case} {c_dtype}: max-norm relative error {err:.3e}"


def test_fused_epilogue_through_the_dispatch_with_other_output_types(cuda_device):
    """FP32 output on a shape whose plan is 256 x 256 outputs per CTA falls back to 128 x 256; BF16 stays."""
    import torch

    M = N = K = 4096
    A, B = make_inputs(M, N, K, seed=68)
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    rows = [0, 255, 256, 2049, M - 1]
    ref = np.stack([oracle.gemm_f32_rows(A, B, r, 1)[0] for r in rows])
    for dtype, tol in ((torch.float32, 2e-5), (torch.bfloat16, 2.0 ** -8)):
        C = torch.full((M, N), float("nan"), dtype=dtype, device=cuda_device)
        api.hgemm_fused(dA, dB, C, 1.0, 0.0)
        torch.cuda.synchronize(cuda_device)
        assert torch.isfinite(C).all()
        got = C[rows].float().cpu().numpy()
        assert np.abs(got - ref).max() / np.abs(ref).max() <= tol, dtype
    assert api.last_device_error() == 0


def test_fused_epilogue_error_codes(cuda_device):
    import ctypes

    import torch

    A, B = make_inputs(128, 128, 128, seed=64)
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    C = torch.empty((128, 128), dtype=torch.float16, device=cuda_device)
    with pytest.raises(_native.HgemmError) as e:
        api.hgemm_fused(dA, dB, C, 1.0, 0.5)  # beta without c_in
    assert e.value.status == _native.ERR_INVALID_ARG
    lib = _native.load()
    assert lib.b200_hgemm_fused(dA.data_ptr(), dB.data_ptr(), C.data_ptr(), 128, 128, 128, None, None) == _native.ERR_INVALID_ARG
    A2, B2 = make_inputs(64, 64, 100, seed=65)  # K % 8 != 0: no tensor-core kernel, so no fused epilogue
    C2 = torch.empty((64, 64), dtype=torch.float16, device=cuda_device)
    with pytest.raises(_native.HgemmError) as e:
        api.hgemm_fused(to_dev(A2, cuda_device), to_dev(B2, cuda_device), C2, 2.0, 0.0)
    assert e.value.status == _native.ERR_UNSUPPORTED
    epi = _native.Epilogue(1.0, 0.0, dA.data_ptr() + 2, None, _native.C_F16)  # bias not 16-byte aligned
    assert lib.b200_hgemm_fused(dA.data_ptr(), dB.data_ptr(), C.data_ptr(), 128, 128, 128, ctypes.byref(epi), None) == _native.ERR_MISALIGNED
    torch.cuda.synchronize(cuda_device)


def test_error_codes_on_device(cuda_device):
    import torch

    lib = _native.load()
    A = torch.zeros(64 * 64 + 8, dtype=torch.float16, device=cuda_device)
    B = torch.zeros(64 * 64, dtype=torch.float16, device=cuda_device)
    C = torch.zeros(64 * 64, dtype=torch.float16, device=cuda_device)
    # a pointer 2 bytes off a 16-byte boundary
    assert lib.b200_hgemm(A.data_ptr() + 2, B.data_ptr(), C.data_ptr(), 64, 64, 64, None) == _native.ERR_MISALIGNED
    # tensor-core variants refuse K % 8 != 0 instead of computing something else
    assert lib.b200_hgemm_ex(A.data_ptr(), B.data_ptr(), C.data_ptr(), 64, 64, 60,
                             ctypes.byref(plan_of(_native.VARIANT_CTA1, 256)), None) == _native.ERR_UNSUPPORTED
    assert lib.b200_hgemm_ex(A.data_ptr(), B.data_ptr(), C.data_ptr(), 64, 64, 64,
                             ctypes.byref(plan_of(_native.VARIANT_CTA1, 96)), None) == _native.ERR_UNSUPPORTED
    # a caller-provided workspace that is too small is reported, not outgrown
    ws = torch.zeros(1 << 17, dtype=torch.uint8, device=cuda_device)
    assert lib.b200_hgemm_set_workspace(ws.data_ptr(), ws.numel()) == 0
    rc = lib.b200_hgemm_ex(A.data_ptr(), B.data_ptr(), C.data_ptr(), 64, 64, 64,
                           ctypes.byref(plan_of(_native.VARIANT_STREAMK, 256, parts=8)), None)
    assert rc == _native.ERR_WORKSPACE
    assert lib.b200_hgemm_set_workspace(None, 0) == 0
    torch.cuda.synchronize()
    assert api.last_device_error() == 0


def test_concurrent_streams_and_threads_do_not_share_scratch(cuda_device):
    """Stream-k GEMMs issued from several host threads on several streams at once: every stream has
    its own partial-tile workspace, so the results are those of the same calls made one by one."""
    import threading

    import torch

    shapes = [(64, 2048, 4096), (128, 1024, 8192), (200, 1032, 1096), (16, 3584, 2048)]
    jobs = []
    for i, (M, N, K) in enumerate(shapes):
        A, B = make_inputs(M, N, K, seed=30 + i, dist="normal")
        dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
        expect = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
        api.b200HgemmStreamK(dA, dB, expect)
        jobs.append((dA, dB, expect, torch.cuda.Stream(device=cuda_device)))
    torch.cuda.synchronize()
    outs = [torch.full_like(j[2], float("nan")) for j in jobs]
    errors = []

    def worker(idx):
        try:
            dA, dB, _, stream = jobs[idx]
            with torch.cuda.stream(stream):
                for _ in range(20):
                    api.b200HgemmStreamK(dA, dB, outs[idx])
            stream.synchronize()
        except Exception as exc:  # surfaced below
            errors.append(exc)

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(len(jobs))]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    torch.cuda.synchronize()
    assert not errors, errors
    assert api.last_device_error() == 0
    for (dA, dB, expect, _), out in zip(jobs, outs):
        assert torch.equal(out, expect)


def test_an_expired_wait_is_reported_and_the_device_stays_usable(cuda_device):
    """Failure detection without a fault: a wait that cannot complete runs into its time limit, the
    kernel returns, the host reads the error word, and the next GEMM on the same context is correct."""
    import time

    import torch

    lib = _native.load()
    assert api.last_device_error() == 0
    t0 = time.perf_counter()
    assert lib.b200_debug_wait_expiry(50, None) == _native.OK  # 50 ms limit
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.04 < waited < 2.0, waited
    assert api.last_device_error() == 1   # reported once ...
    assert api.last_device_error() == 0   # ... and cleared
    assert lib.b200_debug_wait_expiry(0, None) == _native.ERR_INVALID_ARG
    assert lib.b200_debug_wait_expiry(5000, None) == _native.ERR_INVALID_ARG
    A, B = make_inputs(256, 256, 256, seed=40)
    C = run(api.b200Hgemm, A, B, cuda_device)
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), "after an expired wait")


def test_synchronize_reports_an_expired_wait_as_a_status(cuda_device):
    """b200_hgemm_synchronize: waits for one stream and turns a raised error word into B200_HGEMM_ERR_DEVICE_WAIT."""
    import torch

    lib = _native.load()
    stream = torch.cuda.Stream(device=cuda_device)
    assert lib.b200_hgemm_synchronize(stream.cuda_stream) == _native.OK
    assert lib.b200_debug_wait_expiry(20, stream.cuda_stream) == _native.OK
    assert lib.b200_hgemm_synchronize(stream.cuda_stream) == _native.ERR_DEVICE_WAIT
    assert lib.b200_hgemm_synchronize(stream.cuda_stream) == _native.OK   # cleared
    assert api.last_device_error() == 0
    A, B = make_inputs(256, 256, 256, seed=41)
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    C = poisoned(256, 256, cuda_device).view(256, 256)
    with torch.cuda.stream(stream):
        api.b200Hgemm(dA, dB, C)
        api.synchronize(cuda_device)
    assert_close_to_oracle(C.cpu().numpy(), oracle.gemm_f32(A, B), "after a reported wait")


def test_more_streams_than_workspace_slots(cuda_device):
    """The library keeps a stream-k workspace per stream, 64 at most: the 65th stream and every later one
    still gets one (the one used longest ago changes hands), and they can all be released."""
    import torch

    lib = _native.load()
    M, N, K = 96, 1024, 2048
    A, B = make_inputs(M, N, K, seed=42, dist="normal")
    dA, dB = to_dev(A, cuda_device), to_dev(B, cuda_device)
    expect = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
    api.b200HgemmStreamK(dA, dB, expect)
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(device=cuda_device) for _ in range(70)]
    out = torch.empty((M, N), dtype=torch.float16, device=cuda_device)
    for s in streams:
        out.fill_(float("nan"))
        torch.cuda.synchronize()
        with torch.cuda.stream(s):
            api.b200HgemmStreamK(dA, dB, out)
        s.synchronize()
        assert torch.equal(out, expect)
    torch.cuda.synchronize()
    freed = lib.b200_hgemm_release_workspaces()
    assert 1 <= freed <= 64
    assert lib.b200_hgemm_release_workspaces() == 0
    api.b200HgemmStreamK(dA, dB, out)   # allocates afresh
    torch.cuda.synchronize()
    assert torch.equal(out, expect)
    assert api.last_device_error() == 0


@pytest.mark.parametrize("shape", [
    (1, 8, 8), (1, 8, 4096), (4096, 8, 64), (8, 4096, 64), (128, 256, 8), (129, 257 * 8, 72), (16, 16, 65536),
    (40000, 16, 64), (24, 40000, 64), (2304, 2304, 2304), (3000, 1000, 520),
], ids=lambda s: "x".join(map(str, s)))
def test_extreme_aspect_ratios(cuda_device, shape):
    """Degenerate and lopsided shapes through the auto dispatch: one row, eight columns, one k-block of
    eight, very deep k, hundreds of row or column blocks."""
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=50, dist="normal")
    C = run(api.b200Hgemm, A, B, cuda_device)
    assert_close_to_oracle(C, oracle.gemm_f32(A, B), f"auto {shape}")


def test_static_scratch_and_every_variant_on_a_lopsided_shape(cuda_device):
    M, N, K = 72, 1544, 2056
    A, B = make_inputs(M, N, K, seed=51)
    ref = oracle.gemm_f32(A, B)
    for variant, bn in ((_native.VARIANT_CTA1, 64), (_native.VARIANT_CTA1, 256), (_native.VARIANT_CTA2, 128),
                        (_native.VARIANT_CTA2, 256), (_native.VARIANT_STREAMK, 64), (_native.VARIANT_STREAMK, 256),
                        (_native.VARIANT_SIMT, 0)):
        C = run(None, A, B, cuda_device, plan_of(variant, bn))
        assert_close_to_oracle(C, ref, f"variant {variant} bn {bn}")


# ---- the benchmark's own sizes -------------------------------------------------------------
def device_inputs(M, N, K, dist, seed, device):
    """Seeded FP16 operands drawn on the GPU (the host would need minutes for 16384^2 draws): uniform [-1, 1),
    or activations ~ N(0, 1) and weights ~ N(0, 1/K)."""
    import torch

    g = torch.Generator(device=device)
    g.manual_seed(seed)
    if dist == "uniform":
        A = torch.rand((M, K), generator=g, device=device, dtype=torch.float32).mul_(2).sub_(1).half()
        B = torch.rand((N, K), generator=g, device=device, dtype=torch.float32).mul_(2).sub_(1).half()
    else:
        A = torch.randn((M, K), generator=g, device=device, dtype=torch.float32).half()
        B = torch.randn((N, K), generator=g, device=device, dtype=torch.float32).div_(K ** 0.5).half()
    return A, B


def check_sampled_row_blocks(C, dA, hB, row_blocks, what):
    """128-row blocks of C against the oracle: together they cover every column tile and every k-block."""
    import torch

    rows = torch.cat([torch.arange(r, r + 128, device=dA.device) for r in row_blocks])
    ref = oracle.gemm_f32(dA[rows].cpu().numpy(), hB)
    assert_close_to_oracle(C[rows].cpu().numpy(), ref, what)


@pytest.mark.parametrize("plan_name", ["auto", "pairs_512x256", "multicast_512x512", "pairs_256x256"])
def test_square_16384_sampled_rows(cuda_device, plan_name, request):
    """The benchmark's headline shape under every arrangement the dispatch can give it: many tiles per CTA,
    256 k-blocks per tile."""
    import torch

    if plan_name == "multicast_512x512":
        request.getfixturevalue("multicast_on")
    plan = {"auto": None, "pairs_512x256": plan_of(_native.VARIANT_CTA2, 512),
            "multicast_512x512": plan_of(_native.VARIANT_CTA2_MCAST, 512),
            "pairs_256x256": plan_of(_native.VARIANT_CTA2, 256)}[plan_name]
    M = N = K = 16384
    dA, dB = device_inputs(M, N, K, "uniform", 2023, cuda_device)
    C = poisoned(M, N, cuda_device).view(M, N)
    if plan is None:
        api.b200Hgemm(dA, dB, C)
    else:
        api.hgemm_ex(dA, dB, C, plan)
    torch.cuda.synchronize()
    assert api.last_device_error() == 0
    assert torch.isfinite(C).all()
    check_sampled_row_blocks(C, dA, dB.cpu().numpy(), (0, 8192 + 384, M - 128), f"16384^3 {plan_name}")


def test_prefill_shape_sampled_rows(cuda_device):
    """8192 x 28672 x 8192, activations ~ N(0,1), weights ~ N(0, 1/K)."""
    import torch

    M, N, K = 8192, 28672, 8192
    dA, dB = device_inputs(M, N, K, "normal", 2024, cuda_device)
    C = poisoned(M, N, cuda_device).view(M, N)
    api.b200Hgemm(dA, dB, C)
    torch.cuda.synchronize()
    assert api.last_device_error() == 0
    assert torch.isfinite(C).all()
    check_sampled_row_blocks(C, dA, dB.cpu().numpy(), (0, 4096 - 128, M - 128), "prefill")


@pytest.mark.parametrize("NK", [(14336, 4096), (4096, 14336)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("M", [16, 32, 64, 128])
def test_decode_shapes_at_full_size(cuda_device, M, NK):
    """The decode configurations at their true N and K, every row against the oracle, through the dispatch."""
    import torch

    N, K = NK
    dA, dB = device_inputs(M, N, K, "normal", 2025 + M, cuda_device)
    C = poisoned(M, N, cuda_device).view(M, N)
    api.b200Hgemm(dA, dB, C)
    torch.cuda.synchronize()
    assert api.last_device_error() == 0
    ref = oracle.gemm_f32(dA.cpu().numpy(), dB.cpu().numpy())
    assert_close_to_oracle(C.cpu().numpy(), ref, f"decode {M}x{N}x{K} plan {api.select_plan(M, N, K).as_dict()}")


# ---- stacks of matrices ---------------------------------------------------------------------
BATCHED_CASES = [
    # batch, M, N, K, gap in elements between consecutive matrices (0 = dense), B shared?
    (5, 200, 264, 136, 0, False),      # tails in M, N and K
    (64, 128, 128, 64, 0, False),      # many one-tile products, one k-block each
    (40, 512, 512, 128, 0, False),     # enough 256 x 256 tiles for CTA pairs
    (7, 96, 1000, 520, 4096, False),   # gaps between the matrices
    (3, 100, 100, 64, 8, False),       # N % 8 != 0: plain stores
    (6, 48, 512, 256, 0, True),        # one B for the whole stack, A and C dense: one product of batch * M rows
    (4, 64, 256, 128, 1024, True),     # one B, gaps in A and C: product by product
    (3, 40, 48, 100, 0, False),        # K % 8 != 0: product by product on the CUDA-core kernel
    (1, 256, 256, 256, 0, False),
]


@pytest.mark.parametrize("case", BATCHED_CASES, ids=lambda c: f"b{c[0]}-" + "x".join(map(str, c[1:4])) + f"-gap{c[4]}" + ("-sharedB" if c[5] else ""))
def test_batched_products(cuda_device, case):
    """b200_hgemm_batched: every matrix of the stack against the oracle; the gaps between matrices stay untouched."""
    import torch

    batch, M, N, K, gap, shared_b = case
    rng = np.random.default_rng(71)
    A = rng.uniform(-1, 1, size=(batch, M, K)).astype(np.float16)
    B = rng.uniform(-1, 1, size=((1 if shared_b else batch), N, K)).astype(np.float16)

    def stack(x, rows, cols, fill):
        flat = torch.full((x.shape[0] * (rows * cols + gap),), fill, dtype=torch.float16, device=cuda_device)
        view = torch.as_strided(flat, (x.shape[0], rows, cols), (rows * cols + gap, cols, 1))
        view.copy_(torch.from_numpy(x).to(cuda_device))
        return flat, view

    _, dA = stack(A, M, K, 0.0)
    dB = torch.from_numpy(B[0]).to(cuda_device) if shared_b else stack(B, N, K, 0.0)[1]
    c_flat, dC = stack(np.zeros((batch, M, N), dtype=np.float16), M, N, float("nan"))
    dC.fill_(float("nan"))
    api.hgemm_batched(dA, dB, dC)
    torch.cuda.synchronize(cuda_device)
    assert api.last_device_error() == 0
    got = dC.cpu().numpy()
    for i in range(batch):
        assert_close_to_oracle(got[i], oracle.gemm_f32(A[i], B[0 if shared_b else i]), f"batched {case} matrix {i}")
    if gap:
        gaps = torch.as_strided(c_flat, (batch, gap), (M * N + gap, 1), storage_offset=M * N)
        assert torch.isnan(gaps).all(), "the call wrote between the matrices of C"


def test_batched_products_refuse_overlapping_or_misaligned_stacks(cuda_device):
    import torch

    lib = _native.load()
    buf = torch.zeros(1 << 20, dtype=torch.float16, device=cuda_device)
    p = buf.data_ptr()
    M = N = K = 64
    dense = M * K
    assert lib.b200_hgemm_batched(p, p, p, M, N, K, 0, dense, dense, dense, None) == _native.ERR_INVALID_ARG
    assert lib.b200_hgemm_batched(p, p, p, M, N, K, 4, dense - 8, dense, dense, None) == _native.ERR_INVALID_ARG   # A_i overlap
    assert lib.b200_hgemm_batched(p, p, p, M, N, K, 4, dense, dense, dense + 4, None) == _native.ERR_MISALIGNED    # C_i off 16 bytes
    torch.cuda.synchronize()


# ---- B stored K x N row-major -----------------------------------------------------------------
@pytest.mark.parametrize("shape", [
    (128, 64, 64), (128, 256, 64), (128, 256, 128), (256, 256, 256), (384, 512, 320), (200, 264, 136), (16, 1024, 512),
    (100, 14336, 256), (1024, 1024, 1024), (2304, 2560, 512), (4096, 4096, 1024), (520, 264, 8200),
], ids=lambda s: "x".join(map(str, s)))
def test_b_stored_k_by_n_row_major(cuda_device, shape):
    """b200_hgemm_bkn: B as K rows of N halves, read by the MMA as an MN-major operand; the same bits as the
    K-contiguous form on the transposed copy when both run the same tiles, the oracle's tolerance always."""
    import torch

    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=81)          # B is [N, K]
    B_kn = np.ascontiguousarray(B.T)              # the same matrix stored [K, N]
    dA, dB = to_dev(A, cuda_device), to_dev(B_kn, cuda_device)
    flat = poisoned(M, N, cuda_device, extra_rows=4)
    C = flat[: M * N].view(M, N)
    api.hgemm_bkn(dA, dB, C)
    torch.cuda.synchronize(cuda_device)
    assert api.last_device_error() == 0
    assert (flat[M * N:].view(torch.int16).cpu().numpy() == POISON).all()
    assert_close_to_oracle(C.cpu().numpy(), oracle.gemm_f32(A, B), f"B as K x N {shape}")


def test_b_stored_k_by_n_refuses_row_pitches_tma_cannot_take(cuda_device):
    import torch

    lib = _native.load()
    buf = torch.zeros(1 << 16, dtype=torch.float16, device=cuda_device)
    p = buf.data_ptr()
    assert lib.b200_hgemm_bkn(p, p, p, 64, 60, 64, None) == _native.ERR_UNSUPPORTED
    assert lib.b200_hgemm_bkn(p, p, p, 64, 64, 60, None) == _native.ERR_UNSUPPORTED
    assert lib.b200_hgemm_bkn(p, p + 2, p, 64, 64, 64, None) == _native.ERR_MISALIGNED
    torch.cuda.synchronize()
