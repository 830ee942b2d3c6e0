"""The allocation-free stream-k entry point, ``b200_hgemm_streamk_static``.

Some users of this library cannot allocate device memory where they need a GEMM: all memory
belongs to a pool, an allocation's implicit synchronisation would stall a serving loop, or the
host application forbids allocations after start-up. For them the library offers one entry
point whose scratch (the FP32 partial tiles of split k-ranges) is a static 16 MiB device array.
This test calls it through the C ABI twice in a row -- the second call finds the array as the
first one left it -- and compares each result with the ordinary stream-k entry point and with
the CPU oracle, on the tolerance the other parity tests use. It also checks that the call
really allocates nothing, that sizes beyond its stated maximum are refused, and that a wait
that expires inside it can be read back by the caller.
"""
import numpy as np
import pytest

from cuda_hgemm_b200 import _native, api
from oracle import hgemm_oracle as oracle
from tests.helpers import assert_close_to_oracle, make_inputs

pytestmark = pytest.mark.gpu


def call_static(lib, dA, dB, dC, M, N, K):
    import torch

    return lib.b200_hgemm_streamk_static(dA.data_ptr(), dB.data_ptr(), dC.data_ptr(), M, N, K,
                                         torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("shape,dist", [((16, 3584, 1024), "normal"), ((200, 1032, 1096), "uniform"),
                                        ((128, 1024, 3584), "normal")],
                         ids=["skinny", "tails", "deep_k"])
def test_static_scratch_matches_stream_k_on_two_calls_in_a_row(cuda_device, shape, dist):
    import torch

    lib = _native.load()
    M, N, K = shape
    A, B = make_inputs(M, N, K, seed=21, dist=dist)
    ref = oracle.gemm_f32(A, B)
    dA, dB = torch.from_numpy(A).to(cuda_device), torch.from_numpy(B).to(cuda_device)

    expected = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
    api.b200HgemmStreamK(dA, dB, expected)
    torch.cuda.synchronize()
    assert api.last_device_error() == 0
    expected_np = expected.cpu().numpy()
    assert_close_to_oracle(expected_np, ref, "stream-k")

    results = []
    for call in range(2):
        out = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
        free_before, _ = torch.cuda.mem_get_info(cuda_device)
        assert call_static(lib, dA, dB, out, M, N, K) == _native.OK
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(cuda_device)
        if call == 1:
            # set-up (kernel attributes, module data) is behind us: nothing may have been allocated
            assert free_after == free_before
        assert lib.b200_hgemm_streamk_static_last_error() == 0
        got = out.cpu().numpy()
        assert_close_to_oracle(got, ref, f"static call {call}")
        # same products and the same FP32 accumulation, grouped into a different number of k-ranges:
        # the two entry points agree to one FP16 rounding step of each value
        diff = np.abs(got.astype(np.float64) - expected_np.astype(np.float64))
        assert (diff <= 2.0 ** -9 * np.abs(expected_np.astype(np.float64)) + 1e-3 * np.abs(ref).max()).all()
        results.append(got)
    # the array's leftover contents do not leak into the next result
    assert np.array_equal(results[0].view(np.uint16), results[1].view(np.uint16))


def test_static_scratch_refuses_what_does_not_fit(cuda_device):
    import torch

    lib = _native.load()
    buf = torch.zeros(1 << 16, dtype=torch.float16, device=cuda_device)
    p = buf.data_ptr()
    # 129 x 128 row blocks times 128 column blocks > 16384 tiles: refused before anything is touched
    assert lib.b200_hgemm_streamk_static(p, p, p, 129 * 128, 128 * 128, 64, None) == _native.ERR_TOO_LARGE
    assert lib.b200_hgemm_streamk_static(p, p, p, 64, 64, 60, None) == _native.ERR_UNSUPPORTED
    assert lib.b200_hgemm_streamk_static(None, p, p, 64, 64, 64, None) == _native.ERR_INVALID_ARG
    torch.cuda.synchronize()


def test_an_expired_wait_inside_the_static_variant_can_be_read_back(cuda_device):
    """The static variant reports a bounded wait that ran out in the first word of its array; the caller reads
    it with b200_hgemm_streamk_static_last_error(), which allocates nothing either. The expiry is produced
    without any fault: one CTA waits 50 ms on a barrier that nothing arrives on."""
    import torch

    lib = _native.load()
    assert lib.b200_hgemm_streamk_static_last_error() == 0
    assert lib.b200_debug_wait_expiry_static(50, None) == _native.OK
    assert lib.b200_hgemm_streamk_static_last_error() == 1   # reported once ...
    assert lib.b200_hgemm_streamk_static_last_error() == 0   # ... and cleared
    assert api.last_device_error() == 0                      # the other entry points' word is a different one
    # the next call through the static variant starts clean and is correct
    M, N, K = 128, 512, 1024
    A, B = make_inputs(M, N, K, seed=22, dist="normal")
    dA, dB = torch.from_numpy(A).to(cuda_device), torch.from_numpy(B).to(cuda_device)
    out = torch.full((M, N), float("nan"), dtype=torch.float16, device=cuda_device)
    assert call_static(lib, dA, dB, out, M, N, K) == _native.OK
    torch.cuda.synchronize()
    assert lib.b200_hgemm_streamk_static_last_error() == 0
    assert_close_to_oracle(out.cpu().numpy(), oracle.gemm_f32(A, B), "static after an expired wait")
