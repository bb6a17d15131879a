"""GPU test of w4a8_gemm_splitk_static, the split-K entry point for callers that cannot allocate device memory
(serving loops that must not touch the allocator while running, host plugins that were only handed their input and
output buffers).
Its partial sums live in a fixed buffer inside the library, shared by all calls, so the test calls it twice in a
row — with different shapes, so the second call finds the first call's leftovers in the buffer — and compares each
result bit for bit with w4a8_gemm_splitk fed a caller-owned workspace.  Collected last (file name) so that a
stop-at-first-failure run has already executed every other test.
"""
import numpy as np
import pytest
import torch

from conftest import to_dev

pytestmark = pytest.mark.gpu


def _case(oracle, M, N, K, seed):
    X = oracle.make_activations(M, K, seed=seed)
    Wq, sw = oracle.make_weights(N, K, seed=seed + 1)
    xq, xs, _ = oracle.quantize_x_q8(X)
    return xq, xs, Wq, sw


def test_static_scratch_splitk_matches_workspace_splitk_twice_in_a_row(w4a8, oracle, cuda):
    for (M, N, K, splitk) in [(16, 512, 2048, 8), (14, 300, 1024, 0), (16, 512, 2048, 8)]:
        xq, xs, Wq, sw = _case(oracle, M, N, K, seed=7000 + M + N + K)
        d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
        nbytes = w4a8.gemm_splitk_workspace_bytes(M, N, K, splitk)
        assert 0 < nbytes <= w4a8.SPLITK_STATIC_BYTES
        ws = torch.empty(nbytes // 4, dtype=torch.float32, device=cuda)
        Y_ref = torch.empty((M, N), dtype=torch.float32, device=cuda)
        w4a8.launch_gemm_bm16_splitk(d[0], d[1], d[2], d[3], Y_ref, M, N, K, splitk=splitk, workspace=ws)
        for _ in range(2):                                                   # two calls in a row on the shared buffer
            Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=cuda)
            w4a8.launch_gemm_splitk_static(d[0], d[1], d[2], d[3], Y, M, N, K, splitk=splitk)
            w4a8.device_status()
            assert torch.equal(Y, Y_ref)                                      # same bits as the existing entry point
        nsplit = nbytes // (M * N * 4)
        assert np.array_equal(Y_ref.cpu().numpy().view(np.uint32), oracle.gemm_splitk_w4a8(xq, xs, Wq, sw, nsplit).view(np.uint32))


def test_static_scratch_splitk_rejects_what_does_not_fit(w4a8, cuda):
    M, N, K = 4096, 2048, 512                       # 8 splits x 4096 x 2048 x 4 B = 256 MiB > 16 MiB
    assert w4a8.gemm_splitk_workspace_bytes(M, N, K, 8) > w4a8.SPLITK_STATIC_BYTES
    a = torch.zeros(16, dtype=torch.int8, device=cuda)     # never dereferenced: the size check comes first
    with pytest.raises(w4a8.W4A8Error) as ei:
        w4a8.launch_gemm_splitk_static(a, a, a, a, a, M, N, K, splitk=8)
    assert ei.value.code == w4a8.ERR_UNSUPPORTED
    assert "built-in buffer" in str(ei.value) and "caller-owned workspace" in str(ei.value)
