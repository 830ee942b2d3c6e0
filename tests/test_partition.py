"""Row-slab partition and the optional C all-gather, on CPU ranks (gloo, world size 2)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cuda_hgemm_b200.partition import row_slabs


@pytest.mark.parametrize("M,world", [(16384, 8), (8192, 2), (8192, 4), (300, 4), (128, 8), (0, 2), (1000, 3)])
def test_row_slabs_tile_aligned_and_complete(M, world):
    slabs = row_slabs(M, world)
    assert len(slabs) == world
    assert slabs[0][0] == 0 and slabs[-1][1] == M
    for (l0, h0), (l1, h1) in zip(slabs, slabs[1:]):
        assert h0 == l1
    for lo, hi in slabs:
        assert lo <= hi and (lo % 128 == 0 or lo == M)
    heights = [h - l for l, h in slabs]
    # heights differ by at most one tile row block plus the ragged tail of M
    assert max(heights) - min(heights) < 256 or M < 128 * world


def test_c_abi_partition_matches_the_python_rule(native_lib):
    """b200_partition_slab (the rule b200_mg_hgemm applies) and partition.row_slabs are the same function."""
    import ctypes

    for M in (0, 1, 127, 128, 129, 300, 1000, 8192, 16384, 16385, 100000):
        for world in (1, 2, 3, 4, 7, 8):
            expected = row_slabs(M, world)
            for index in range(world):
                row0, rows = ctypes.c_size_t(), ctypes.c_size_t()
                assert native_lib.b200_partition_slab(M, world, index, ctypes.byref(row0), ctypes.byref(rows)) == 0
                assert (row0.value, row0.value + rows.value) == expected[index], (M, world, index)
    row0, rows = ctypes.c_size_t(), ctypes.c_size_t()
    assert native_lib.b200_partition_slab(1024, 0, 0, ctypes.byref(row0), ctypes.byref(rows)) == -1
    assert native_lib.b200_partition_slab(1024, 2, 2, ctypes.byref(row0), ctypes.byref(rows)) == -1


def test_benchmark_partitions():
    assert [h - l for l, h in row_slabs(16384, 8)] == [2048] * 8
    assert [h - l for l, h in row_slabs(8192, 4)] == [2048] * 4


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cuda_hgemm_b200 import multi_gpu
        from oracle import hgemm_oracle as oracle
        from tests.helpers import make_inputs

        A, B = make_inputs(M, N, K, seed=77)  # every rank regenerates the same inputs from the seed
        lo, hi = multi_gpu.rank_slab(M, rank, world)
        # stand-in for the device multiply of this rank's slab (no GPU here): the CPU checker
        slab = oracle.gemm_f16(A[lo:hi], B, threads=2) if hi > lo else np.zeros((0, N), np.float16)
        full = multi_gpu.allgather_c(torch.from_numpy(slab.copy()), M, N)
        expect = oracle.gemm_f16(A, B, threads=2)
        ok = np.array_equal(full.numpy().view(np.uint16), expect.view(np.uint16))
        with open(os.path.join(result_dir, f"rank{rank}.txt"), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("M", [512, 300])
def test_allgather_of_slabs_rebuilds_c_on_every_rank(tmp_path, M):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), M, 96, 64, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"rank{r}.txt").read_text() == "ok"


def _exchange_worker(rank, world, port, N, K, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cuda_hgemm_b200 import multi_gpu
        from tests.helpers import make_inputs

        _, B = make_inputs(8, N, K, seed=78)  # the whole of B, as every rank's host memory holds it
        lo, hi = multi_gpu.share_of_b(N, rank, world)
        device_copy = torch.full((N, K), float("nan"), dtype=torch.float16)  # stand-in for the device buffer
        device_copy[lo:hi] = torch.from_numpy(B[lo:hi])                      # the share this rank uploads
        multi_gpu.exchange_b(device_copy, rank, world)
        ok = np.array_equal(device_copy.numpy().view(np.uint16), B.view(np.uint16))
        with open(os.path.join(result_dir, f"exchange{rank}.txt"), "w") as f:
            f.write("ok" if ok else "mismatch")
    finally:
        dist.destroy_process_group()


def test_exchange_of_b_shares_rebuilds_b_on_every_rank(tmp_path):
    """Each rank holds 1/world of B on its device; the in-place all-gather completes every copy."""
    world = 2
    mp.spawn(_exchange_worker, args=(world, _free_port(), 192, 64, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert (tmp_path / f"exchange{r}.txt").read_text() == "ok"


def test_shares_of_b_are_equal_and_complete():
    from cuda_hgemm_b200 import multi_gpu

    assert [multi_gpu.share_of_b(16384, r, 8) for r in range(8)] == [(r * 2048, (r + 1) * 2048) for r in range(8)]
    with pytest.raises(ValueError):
        multi_gpu.share_of_b(1000, 0, 3)

