"""The allocation-free argmax entry point (collected last on purpose: if it fails, every other test has run).

ie_b200_argmax_static serves hosts that cannot cudaMalloc scratch at call time (all device memory committed at
start-up, or a call site where the CUDA allocator must not be entered): its partials live in a fixed array
inside the library. It must give exactly what ie_b200_argmax gives with caller-provided scratch, call after
call (the array keeps the previous call's contents), and refuse more rows than the array holds."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_argmax_static_matches_argmax(cuda, lib):
    import torch

    from amd_c_b200._lib import check

    rng = np.random.default_rng(77)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (T, n) in enumerate([(3, 128256), (64, 1000)]):  # two calls in a row, different shapes, shared scratch
        x = rng.standard_normal((T, n)).astype(np.float32)
        x[0, 5] = x[0, n - 7] = 60.0  # a tie: the smaller index must win
        d_x = torch.from_numpy(x).to(cuda)
        part = torch.empty(lib.ie_b200_argmax_part_bytes(T), dtype=torch.uint8, device=cuda)
        want = torch.empty((T, 2), dtype=torch.int32, device=cuda)
        got = torch.full((T, 2), -1, dtype=torch.int32, device=cuda)
        check(lib.ie_b200_argmax(d_x.data_ptr(), n, want.data_ptr(), T, n * 4, 8, part.data_ptr(), stream))
        check(lib.ie_b200_argmax_static(d_x.data_ptr(), n, got.data_ptr(), T, n * 4, 8, stream))
        torch.cuda.synchronize()
        assert torch.equal(got, want), call  # index and probability bits: the same kernels, so exactly equal
        assert int(got[0, 0]) == 5
        assert (got[:, 0].cpu().numpy() == x.argmax(axis=1)).all()


def test_argmax_static_refuses_too_many_rows(cuda, lib):
    import torch

    mx = lib.ie_b200_argmax_static_max_rows()
    assert mx == 64
    x = torch.zeros((mx + 1, 8), dtype=torch.float32, device=cuda)
    out = torch.zeros((mx + 1, 2), dtype=torch.int32, device=cuda)
    assert lib.ie_b200_argmax_static(x.data_ptr(), 8, out.data_ptr(), mx + 1, 32, 8, None) == -2
    assert b"64" in lib.ie_b200_last_error()
