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


@pytest.mark.parametrize("M,N,K,splitk,sd,gemm_kernel", [
    (16, 256, 1024, 1, 0, 1),        # one split: no partial sums at all, the plain GEMM writes Y
    (16, 512, 2048, 4, 1, 1),        # fp16 scales
    (12, 384, 1024, 3, 0, 0),        # the fp16-operand GEMM kernel
])
def test_static_scratch_splitk_more_cases_and_no_allocation(w4a8, oracle, cuda, M, N, K, splitk, sd, gemm_kernel):
    """More corners of the same comparison, and the point of the entry: device memory in use is the same before and
    after the calls (cudaMemGetInfo through torch; nothing else runs in between)."""
    X = oracle.make_activations(M, K, seed=7100 + M + N)
    Wq, sw = oracle.make_weights(N, K, seed=7101 + M + N, scale_dtype=sd)
    xq, xs, _ = oracle.quantize_x_q8(X)
    d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
    nbytes = w4a8.gemm_splitk_workspace_bytes(M, N, K, splitk)
    ws = torch.empty(max(nbytes, 16) // 4, dtype=torch.float32, device=cuda)
    Y_ref = torch.empty((M, N), dtype=torch.float32, device=cuda)
    Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=cuda)
    w4a8.config("gemm_kernel", gemm_kernel)
    try:
        w4a8.launch_gemm_bm16_splitk(d[0], d[1], d[2], d[3], Y_ref, M, N, K, scale_dtype=sd, splitk=splitk, workspace=ws)
        w4a8.launch_gemm_splitk_static(d[0], d[1], d[2], d[3], Y, M, N, K, scale_dtype=sd, splitk=splitk)   # first call set-up done
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        for _ in range(2):
            Y.fill_(float("nan"))
            w4a8.launch_gemm_splitk_static(d[0], d[1], d[2], d[3], Y, M, N, K, scale_dtype=sd, splitk=splitk)
            torch.cuda.synchronize()
            assert torch.equal(Y, Y_ref)
        free1, _ = torch.cuda.mem_get_info()
        assert free1 == free0
        w4a8.device_status()
    finally:
        w4a8.config("gemm_kernel", 1)
    nsplit = max(1, nbytes // (M * N * 4))
    assert np.array_equal(Y_ref.cpu().numpy().view(np.uint32), oracle.gemm_splitk_w4a8(xq, xs, Wq, sw, nsplit).view(np.uint32))


def test_splitk_entries_refuse_absurd_split_counts(w4a8, cuda):
    a = torch.zeros(64, dtype=torch.int8, device=cuda)      # never dereferenced: the argument check comes first
    for splitk in (2 ** 31 - 1, 2 ** 31 - 64, 100000):
        assert w4a8.gemm_splitk_workspace_bytes(16, 128, 1024, splitk) == 0
        with pytest.raises(w4a8.W4A8Error) as ei:
            w4a8.launch_gemm_splitk_static(a, a, a, a, a, 16, 128, 1024, splitk=splitk)
        assert ei.value.code == w4a8.ERR_ARG and "splitk" in str(ei.value)
        with pytest.raises(w4a8.W4A8Error) as ei:
            w4a8.launch_gemm_bm16_splitk(a, a, a, a, a, 16, 128, 1024, splitk=splitk, workspace=a)
        assert ei.value.code == w4a8.ERR_ARG and "splitk" in str(ei.value)


_FIRST_CALL_UNDER_CAPTURE = r'''
import os, sys
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, os.path.join(ROOT, "oracle"))
import numpy as np, torch
from conftest import load_package, to_dev
import oracle as O
w = load_package(); w.lib()
dev = torch.device("cuda", 0)
M, N, K = 16, 256, 1024
X = O.make_activations(M, K, seed=1); Wq, sw = O.make_weights(N, K, seed=2); xq, xs, _ = O.quantize_x_q8(X)
d = [to_dev(a, dev) for a in (xq, xs, Wq, sw)]
Y = torch.zeros((M, N), dtype=torch.float32, device=dev)
s = torch.cuda.Stream()
torch.cuda.synchronize()
g = torch.cuda.CUDAGraph()
refused = None
with torch.cuda.stream(s):
    g.capture_begin()
    try:
        w.launch_gemm_splitk_static(d[0], d[1], d[2], d[3], Y, M, N, K, splitk=4, stream=s.cuda_stream)
    except w.W4A8Error as e:
        refused = (e.code, str(e))
    g.capture_end()
torch.cuda.synchronize()
assert refused is not None and refused[0] == w.ERR_UNSUPPORTED and "captured" in refused[1], refused
# outside a capture the first call is fine, and the context is intact
w.launch_gemm_splitk_static(d[0], d[1], d[2], d[3], Y, M, N, K, splitk=4)
torch.cuda.synchronize(); w.device_status()
ref = O.gemm_splitk_w4a8(xq, xs, Wq, sw, 4)
assert np.array_equal(Y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
print("capture refusal ok")
'''


def test_static_scratch_first_call_under_stream_capture_is_refused(tmp_path):
    """The first call on a device looks up the built-in buffer, which must not happen while the stream is being captured:
    it is refused with a clear error, nothing is enqueued, and a later call outside the capture works.  Runs in a child
    process so that it really is the process's first call."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "first_call.py"
    script.write_text("ROOT = %r\n" % root + _FIRST_CALL_UNDER_CAPTURE)
    r = subprocess.run([sys.executable, str(script)], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    assert "capture refusal ok" in r.stdout
