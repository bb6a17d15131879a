"""quantize_x fused into its producers: RMSNorm -> quantize and SwiGLU / GeGLU -> quantize in one kernel each.

Bitwise bar: the fused entry equals the reference's OWN two kernels run one after the other (launch_rmsnorm* or
launch_swiglu / launch_geglu, then launch_quantize_x_q8; rebuilt for sm_100a in oracle/_ref) in xq, xs, xsum and
in the optional fp32 intermediate.  Against the CPU oracle the fp32 intermediate agrees to a few ulp (the GPU's
rsqrtf / expf / tanhf are not the C library's), so there the integers are compared with a tolerance that is
written down below.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import to_dev

pytestmark = pytest.mark.gpu

Y_RTOL = 4e-6            # fp32 intermediate, fused kernel vs CPU oracle: |dy| <= Y_RTOL * max|y| of the row
Q_MISMATCH_FRAC = 5e-3   # fraction of int8 outputs that may differ (by exactly 1) from the CPU oracle's


@pytest.fixture(scope="module")
def ref(oracle):
    path = oracle.ref_kernels_path()
    if path is None:
        pytest.skip("oracle/_ref/libref_kernels.so not built (needs the reference tree at build time)")
    lib = ctypes.CDLL(path)
    for name in ("ref_quantize_x_q8", "ref_rmsnorm", "ref_glu"):
        getattr(lib, name).restype = ctypes.c_int
    return lib


def P(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def outputs(S, K, cuda, with_y=True):
    return (torch.full((S, K), float("nan"), dtype=torch.float32, device=cuda) if with_y else None,
            torch.empty((S, K), dtype=torch.int8, device=cuda),
            torch.empty((S, K // 32), dtype=torch.float32, device=cuda),
            torch.empty((S, K // 32), dtype=torch.int32, device=cuda))


def check_against_oracle(oracle, Yo, got):
    """got = (Y, xq, xs, xsum) numpy arrays of the fused kernel; Yo the oracle's fp32 intermediate."""
    Y, xq, xs, xsum = got
    scale = np.max(np.abs(Yo), axis=1, keepdims=True) + 1e-30
    assert np.max(np.abs(Y - Yo) / scale) < Y_RTOL
    xq_o, xs_o, _ = oracle.quantize_x_q8(Yo)
    assert np.allclose(xs, xs_o, rtol=1e-5, atol=0)
    diff = np.abs(xq.astype(np.int32) - xq_o.astype(np.int32))
    assert diff.max() <= 1 and np.mean(diff != 0) < Q_MISMATCH_FRAC
    # and the fused integers are exactly the quantization of the fused kernel's own fp32 intermediate
    xq_s, xs_s, xsum_s = oracle.quantize_x_q8(Y)
    assert np.array_equal(xq, xq_s) and np.array_equal(xs.view(np.uint32), xs_s.view(np.uint32)) and np.array_equal(xsum, xsum_s)


@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("rows,hh", [(1, 5120), (3, 3840), (16, 1024), (5, 160), (2, 15360)])
def test_rmsnorm_quantize(w4a8, oracle, cuda, request, rows, hh, variant):
    rng = np.random.default_rng(1000 + rows + hh + variant)
    X = (rng.normal(0, 1.5, size=(rows, hh)) * rng.lognormal(0, 1, size=(rows, 1))).astype(np.float32)
    X[0, 32:64] = 0.0
    W = rng.normal(0.0 if variant == 1 else 1.0, 0.2, size=hh).astype(np.float32)
    eps = 1e-6
    X_d, W_d = to_dev(X, cuda), to_dev(W, cuda)
    Y, xq, xs, xsum = outputs(rows, hh, cuda)
    w4a8.launch_rmsnorm_quantize_x_q8(X_d, None if variant == 2 else W_d, eps, variant, Y, xq, xs, xsum, hh, rows)
    torch.cuda.synchronize()
    got = (Y.cpu().numpy(), xq.cpu().numpy(), xs.cpu().numpy(), xsum.cpu().numpy())
    check_against_oracle(oracle, oracle.rmsnorm(X, W, eps, variant), got)
    # without the fp32 copy: same integers
    _, xq2, xs2, xsum2 = outputs(rows, hh, cuda, with_y=False)
    w4a8.launch_rmsnorm_quantize_x_q8(X_d, None if variant == 2 else W_d, eps, variant, None, xq2, xs2, xsum2, hh, rows)
    torch.cuda.synchronize()
    assert torch.equal(xq2, xq) and torch.equal(xs2, xs) and torch.equal(xsum2, xsum)
    # bitwise: the reference's own kernels, one after the other
    ref = request.getfixturevalue("ref")
    Yr, xqr, xsr, xsumr = outputs(rows, hh, cuda)
    assert ref.ref_rmsnorm(P(X_d), P(W_d), P(Yr), rows, hh, ctypes.c_float(eps), variant, None) == 0
    assert ref.ref_quantize_x_q8(P(Yr), P(xqr), P(xsr), P(xsumr), hh, rows, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(Yr.view(torch.int32), Y.view(torch.int32))
    assert torch.equal(xqr, xq) and torch.equal(xsr.view(torch.int32), xs.view(torch.int32)) and torch.equal(xsumr, xsum)


@pytest.mark.parametrize("act", [0, 1])
@pytest.mark.parametrize("S,IN", [(1, 17408), (4, 768), (9, 96), (16, 15360)])
def test_glu_quantize(w4a8, oracle, cuda, request, S, IN, act):
    rng = np.random.default_rng(2000 + S + IN + act)
    G = rng.normal(0, 2.0, size=(S, IN)).astype(np.float32)
    U = rng.normal(0, 1.0, size=(S, IN)).astype(np.float32)
    G[0, :32] = 0.0                                                    # a zero block: q = 0, d = 0
    G[0, 40] = -30.0; G[0, 41] = 30.0                                  # saturated ends of the activation
    G_d, U_d = to_dev(G, cuda), to_dev(U, cuda)
    Y, xq, xs, xsum = outputs(S, IN, cuda)
    w4a8.launch_glu_quantize_x_q8(G_d, U_d, act, Y, xq, xs, xsum, IN, S)
    torch.cuda.synchronize()
    got = (Y.cpu().numpy(), xq.cpu().numpy(), xs.cpu().numpy(), xsum.cpu().numpy())
    check_against_oracle(oracle, oracle.glu(G, U, act), got)
    assert np.all(got[1][0, :32] == 0) and got[2][0, 0] == 0.0
    _, xq2, xs2, xsum2 = outputs(S, IN, cuda, with_y=False)
    w4a8.launch_glu_quantize_x_q8(G_d, U_d, act, None, xq2, xs2, xsum2, IN, S)
    torch.cuda.synchronize()
    assert torch.equal(xq2, xq) and torch.equal(xs2, xs) and torch.equal(xsum2, xsum)
    ref = request.getfixturevalue("ref")
    Yr, xqr, xsr, xsumr = outputs(S, IN, cuda)
    assert ref.ref_glu(P(G_d), P(U_d), P(Yr), ctypes.c_long(S * IN), act, None) == 0
    assert ref.ref_quantize_x_q8(P(Yr), P(xqr), P(xsr), P(xsumr), IN, S, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(Yr.view(torch.int32), Y.view(torch.int32))
    assert torch.equal(xqr, xq) and torch.equal(xsr.view(torch.int32), xs.view(torch.int32)) and torch.equal(xsumr, xsum)


def test_fused_then_gemv_equals_unfused_chain(w4a8, oracle, cuda):
    """norm -> quantize -> GEMV through the fused entry gives the bits of quantize_x on the fused kernel's fp32 output."""
    rows, hh, N = 1, 5120, 512
    rng = np.random.default_rng(7)
    X = rng.normal(0, 1, size=(rows, hh)).astype(np.float32)
    W = rng.normal(0, 0.1, size=hh).astype(np.float32)
    Wq, sw = oracle.make_weights(N, hh, seed=5)
    Y, xq, xs, xsum = outputs(rows, hh, cuda)
    w4a8.launch_rmsnorm_quantize_x_q8(to_dev(X, cuda), to_dev(W, cuda), 1e-6, 1, Y, xq, xs, xsum, hh, rows)
    out = torch.empty((rows, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemv_w4a8_sb(xq, xs, to_dev(Wq, cuda), to_dev(sw, cuda), out, hh, N, rows)
    torch.cuda.synchronize()
    xq_o, xs_o, _ = oracle.quantize_x_q8(Y.cpu().numpy())
    assert np.array_equal(out.cpu().numpy().view(np.uint32), oracle.gemv_b200_order(xq_o, xs_o, Wq, sw).view(np.uint32))


def test_fused_entries_reject_bad_arguments(w4a8, cuda):
    X = torch.zeros((1, 64), dtype=torch.float32, device=cuda)
    xq = torch.empty((1, 64), dtype=torch.int8, device=cuda)
    xs = torch.empty((1, 2), dtype=torch.float32, device=cuda)
    with pytest.raises(w4a8.W4A8Error):
        w4a8.launch_rmsnorm_quantize_x_q8(X, X, 1e-6, 3, None, xq, xs, None, 64, 1)        # unknown variant
    with pytest.raises(w4a8.W4A8Error):
        w4a8.launch_rmsnorm_quantize_x_q8(X, None, 1e-6, 0, None, xq, xs, None, 64, 1)     # scale missing
    with pytest.raises(w4a8.W4A8Error):
        w4a8.launch_rmsnorm_quantize_x_q8(X, X, 1e-6, 0, None, xq, xs, None, 48, 1)        # not a multiple of 32
    with pytest.raises(w4a8.W4A8Error):
        w4a8.launch_glu_quantize_x_q8(X, X, 2, None, xq, xs, None, 64, 1)                  # unknown activation
    w4a8.launch_glu_quantize_x_q8(X, X, 0, None, xq, xs, None, 64, 0)                      # S = 0: nothing to do
