"""The reference's OWN kernels, rebuilt for sm_100a (oracle/_ref/libref_kernels.so, built from the reference
headers in place by oracle/Makefile), run beside the oracle and beside this library on the same inputs.

This is what pins the oracle: its GEMV-order and MMQ-order restatements must reproduce the reference
kernels bit for bit, and its quantizer must reproduce quantize_x_q8_kernel exactly.  It also checks the
equalities the reference's own tools assert between its variants (tools/test_sb_vs_gemm_batch.cu,
tools/probe_mlp_vs_sb.cu, tests/test_mmq_tmpl.cu:59-68, tools/r25_raster_gate.cu:98-122).
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import to_dev
from test_gpu_parity import make_case, rel_err, REL_TOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref(oracle):
    path = oracle.ref_kernels_path()
    if path is None:
        pytest.skip("oracle/_ref/libref_kernels.so not built (needs the reference tree at build time)")
    lib = ctypes.CDLL(path)
    for name in ("ref_quantize_x_q8", "ref_gemv_w4a8", "ref_gemv_w4a8_mlp2", "ref_gemv_w4a8_sb", "ref_gemm_batch_w4a8",
                 "ref_gemm_mma_w4a8", "ref_gemm_mmq_w4a8", "ref_gemm_mmq_256x64", "ref_gemm_mmq_raster_w4a8",
                 "ref_gemm_bm16_splitk"):
        getattr(lib, name).restype = ctypes.c_int
    return lib


def P(t):
    return ctypes.c_void_p(t.data_ptr())


def test_reference_quantize_equals_oracle_and_library(ref, w4a8, oracle, cuda):
    for S, K in [(1, 1024), (5, 1024), (16, 5120), (129, 4096)]:
        X = oracle.make_activations(S, K, seed=S * 7 + K, outliers=True)
        X[0, 32:64] = 0.0
        X_d = to_dev(X, cuda)
        outs = []
        for which in ("ref", "lib"):
            xq = torch.empty((S, K), dtype=torch.int8, device=cuda)
            xs = torch.empty((S, K // 32), dtype=torch.float32, device=cuda)
            xsum = torch.empty((S, K // 32), dtype=torch.int32, device=cuda)
            if which == "ref":
                assert ref.ref_quantize_x_q8(P(X_d), P(xq), P(xs), P(xsum), K, S, None) == 0
            else:
                w4a8.launch_quantize_x_q8(X_d, xq, xs, xsum, K, S, stream=0)
            torch.cuda.synchronize()
            outs.append((xq.cpu().numpy(), xs.cpu().numpy(), xsum.cpu().numpy()))
        o = oracle.quantize_x_q8(X)
        for got in outs:
            assert np.array_equal(got[0], o[0])
            assert np.array_equal(got[1].view(np.uint32), o[1].view(np.uint32))
            assert np.array_equal(got[2], o[2])


@pytest.mark.parametrize("scale_dtype", [0, 1])
@pytest.mark.parametrize("IN,OUT,S", [(1024, 256, 1), (3584, 1024, 1), (1024, 4096, 5), (5120, 512, 16), (160, 37, 8)])
def test_reference_gemv_family(ref, w4a8, oracle, cuda, IN, OUT, S, scale_dtype):
    xq, xs, Wq, sw = make_case(oracle, S, OUT, IN, seed=IN + OUT + S, scale_dtype=scale_dtype)
    d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
    xsum = torch.zeros((S, IN // 32), dtype=torch.int32, device=cuda)

    def run(fn, *args):
        Y = torch.full((S, OUT), float("nan"), dtype=torch.float32, device=cuda)
        assert fn(*[a(Y) if callable(a) else a for a in args]) == 0
        torch.cuda.synchronize()
        return Y.cpu().numpy()

    y_plain = run(ref.ref_gemv_w4a8, P(d[0]), P(d[1]), P(xsum), P(d[2]), P(d[3]), P, IN, OUT, S, scale_dtype, None)
    y_mlp = run(ref.ref_gemv_w4a8_mlp2, P(d[0]), P(d[1]), P(xsum), P(d[2]), P(d[3]), P, IN, OUT, S, scale_dtype, None)
    y_sb = run(ref.ref_gemv_w4a8_sb, P(d[0]), P(d[1]), P(d[2]), P(d[3]), P, IN, OUT, S, scale_dtype, None)
    y_gb = run(ref.ref_gemm_batch_w4a8, P(d[0]), P(d[1]), P(d[2]), P(d[3]), P, IN, OUT, S, scale_dtype, None)
    o = oracle.gemv_w4a8(xq, xs, Wq, sw)
    for y in (y_plain, y_mlp, y_sb, y_gb):                 # the reference's family is bit-identical per row ...
        assert np.array_equal(y.view(np.uint32), o.view(np.uint32))   # ... and the oracle restates it exactly
    Y = torch.empty((S, OUT), dtype=torch.float32, device=cuda)
    w4a8.launch_gemv_w4a8_sb(d[0], d[1], d[2], d[3], Y, IN, OUT, S, scale_dtype, stream=0)
    torch.cuda.synchronize()
    assert rel_err(Y.cpu().numpy(), y_plain) < REL_TOL     # this library vs the reference kernel itself


@pytest.mark.parametrize("scale_dtype", [0, 1])
@pytest.mark.parametrize("M,N,K", [(128, 128, 512), (200, 300, 256), (129, 140, 160), (513, 3840, 1024)])
def test_reference_gemm_family(ref, w4a8, oracle, cuda, M, N, K, scale_dtype):
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=M + N + K, scale_dtype=scale_dtype, outliers=True)
    d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
    outs = {}
    for name, fn, extra in (("mmq", ref.ref_gemm_mmq_w4a8, ()), ("mmq256x64", ref.ref_gemm_mmq_256x64, ()),
                            ("mma", ref.ref_gemm_mma_w4a8, ()), ("raster1", ref.ref_gemm_mmq_raster_w4a8, (1, 1)),
                            ("raster2", ref.ref_gemm_mmq_raster_w4a8, (2, 8))):
        Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=cuda)
        if extra:
            rc = fn(P(d[0]), P(d[1]), P(d[2]), P(d[3]), P(Y), M, N, K, scale_dtype, extra[0], extra[1], None)
        else:
            rc = fn(P(d[0]), P(d[1]), P(d[2]), P(d[3]), P(Y), M, N, K, scale_dtype, None)
        assert rc == 0
        torch.cuda.synchronize()
        outs[name] = Y.cpu().numpy()
    o = oracle.gemm_mmq_w4a8(xq, xs, Wq, sw)
    for name, y in outs.items():
        assert np.array_equal(y.view(np.uint32), o.view(np.uint32)), name      # oracle == every reference GEMM variant
    Y = torch.empty((M, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemm_mmq_w4a8(d[0], d[1], d[2], d[3], Y, M, N, K, scale_dtype, stream=0)
    w4a8.device_status()
    assert np.array_equal(Y.cpu().numpy().view(np.uint32), outs["mmq"].view(np.uint32))   # this library == reference MMQ, bitwise


def test_reference_splitk(ref, w4a8, oracle, cuda):
    M, N, K = 16, 512, 2048
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=31)
    d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
    Yr = torch.empty((M, N), dtype=torch.float32, device=cuda)
    assert ref.ref_gemm_bm16_splitk(P(d[0]), P(d[1]), P(d[2]), P(d[3]), P(Yr), M, N, K, 0, None) == 0
    torch.cuda.synchronize()
    nbytes = w4a8.gemm_splitk_workspace_bytes(M, N, K, 0)
    ws = torch.empty(max(nbytes, 16) // 4, dtype=torch.float32, device=cuda)
    Y = torch.empty((M, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemm_bm16_splitk(d[0], d[1], d[2], d[3], Y, M, N, K, splitk=0, workspace=ws, stream=0)
    w4a8.device_status()
    nsplit = max(1, nbytes // (M * N * 4))
    assert np.array_equal(Yr.cpu().numpy().view(np.uint32), oracle.gemm_splitk_w4a8(xq, xs, Wq, sw, nsplit).view(np.uint32))
    assert np.array_equal(Y.cpu().numpy().view(np.uint32), Yr.cpu().numpy().view(np.uint32))


def test_reference_unit_test_runs_against_the_dropin_library(oracle):
    """The reference's own tests/test_w4a8.cu, compiled unmodified against this repository's shim launchers
    (oracle/reftest_w4a8_dropin.cu): its gates are xq and xsum mismatches == 0 and |Y - fp64 golden| < 1e-2."""
    import os
    import subprocess
    exe = os.path.join(os.path.dirname(oracle.__file__), "_ref", "reftest_w4a8_dropin")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/reftest_w4a8_dropin not built (needs the reference tree at build time)")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "[test_w4a8] PASS" in r.stdout and "FAIL" not in r.stdout
    assert r.stdout.count("xq_mis=0 xsum_mis=0") == 4


@pytest.mark.parametrize("name,verdict", [("gemm_mmq", "[test_gemm_mmq] PASS"), ("gemm_mma", "[test_gemm_mma] PASS"),
                                          ("mmq_tmpl", "[test_mmq_tmpl] PASS")])
def test_reference_gemm_tests_run_against_the_dropin_library(oracle, name, verdict):
    """The reference's own tests/test_gemm_mmq.cu, test_gemm_mma.cu and test_mmq_tmpl.cu, compiled unmodified with this
    repository's headers standing in for kernels/*.cuh (oracle/Makefile, rule $(REFTESTS)).  Their gates: GEMM against
    launch_gemv_w4a8 within 1e-5 of the output rms, 30 runs bitwise identical, and the template launcher bitwise equal
    to launch_gemm_mmq_w4a8_kt (tests/test_gemm_mmq.cu:28-34, tests/test_mmq_tmpl.cu:60-67)."""
    import os
    import subprocess
    exe = os.path.join(os.path.dirname(oracle.__file__), "_ref", "reftest_" + name)
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/reftest_%s not built (needs the reference tree at build time)" % name)
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert verdict in r.stdout and "FAIL" not in r.stdout


def test_dropin_device_helpers(oracle):
    """w4a8_pk and mmq_unpack4v of the drop-in headers (kernels/gemv_w4a8.cuh:16-21, kernels/gemm_mmq.cuh:25-28 in the
    reference) over all 65536 inputs (oracle/reftest_unpack.cu)."""
    import os
    import subprocess
    exe = os.path.join(os.path.dirname(oracle.__file__), "_ref", "reftest_unpack")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/reftest_unpack not built")
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "[reftest_unpack] PASS" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]
