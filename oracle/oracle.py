"""numpy/ctypes front end of the CPU oracle (liboracle.so) plus the seeded synthetic-input generators.

TEST INFRASTRUCTURE ONLY.  Imported by tests/, by __graft_entry__.smoke() and by bench.py's
cpu_baseline / --impl reference legs; never by the shipped library or its Python binding.

The arithmetic lives in w4a8_oracle.c (each function cites the reference file:line it restates).  The
generators below produce the input distributions the benchmark configurations name: int4 weights uniform in
[-8, 7] packed two per byte in the reference layout, group-32 fp32 scales |N(0, 0.02)|/7, activations
N(0, 1) (optionally 1 % of entries scaled 20x), all from numpy's PCG64 with an explicit seed.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libref_kernels.so")
# the reference checkout: W4A8_REFERENCE_DIR, else a directory "reference" beside this repository
_REF_TREE = os.environ.get("W4A8_REFERENCE_DIR") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
QBLK = 32
_lib = None


def build(force=False):
    """Compiles liboracle.so (and, when the reference tree is present, _ref/libref_kernels.so)."""
    src = os.path.join(_HERE, "w4a8_oracle.c")
    stale = force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if stale or (os.path.isdir(os.path.join(_REF_TREE, "kernels")) and not os.path.exists(_REF_PATH)):
        if os.path.exists("/usr/bin/make") and os.path.exists("/usr/bin/gcc"):
            subprocess.run(["make", "-C", _HERE, "REF=" + _REF_TREE] + (["-B"] if force else []), check=True, capture_output=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        l = ctypes.CDLL(_LIB_PATH)
        l.oracle_max_threads.restype = ctypes.c_int
        l.oracle_lcg_frand.restype = ctypes.c_float
        _lib = l
    return _lib


def ref_kernels_path():
    """Path of the reference's own CUDA kernels rebuilt for sm_100a, or None if not built."""
    return _REF_PATH if os.path.exists(_REF_PATH) else None


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def max_threads():
    return int(lib().oracle_max_threads())


def set_threads(n):
    lib().oracle_set_threads(int(n))


def lcg_fill(n, mul, seed):
    """n floats from the reference tests' LCG (tests/test_w4a8.cu:16); returns (array, new_seed)."""
    out = np.empty(n, dtype=np.float32)
    s = ctypes.c_uint32(seed)
    lib().oracle_lcg_fill(_p(out), ctypes.c_size_t(n), ctypes.c_float(mul), ctypes.byref(s))
    return out, s.value


def quantize_x_q8(X):
    """X[S,IN] float32 -> (xq int8 [S,IN], xs float32 [S,IN/32], xsum int32 [S,IN/32])."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    S, IN = X.shape
    assert IN % QBLK == 0
    xq = np.empty((S, IN), dtype=np.int8)
    xs = np.empty((S, IN // QBLK), dtype=np.float32)
    xsum = np.empty((S, IN // QBLK), dtype=np.int32)
    lib().oracle_quantize_x_q8(_p(X), _p(xq), _p(xs), _p(xsum), IN, S)
    return xq, xs, xsum


def rmsnorm(X, W, eps, variant=0):
    """RMSNorm in the reference's reduction order (variant 0: * W, 1: * (1 + W), 2: no scale); float32 [rows, hh]."""
    X = np.ascontiguousarray(X, dtype=np.float32)
    rows, hh = X.shape
    Wc = np.ascontiguousarray(W if W is not None else np.zeros(hh), dtype=np.float32)
    Y = np.empty_like(X)
    lib().oracle_rmsnorm(_p(X), _p(Wc), _p(Y), rows, hh, ctypes.c_float(eps), variant)
    return Y


def glu(G, U, act=0):
    """SwiGLU (act 0) or GeGLU (act 1) of float32 arrays of equal shape."""
    G = np.ascontiguousarray(G, dtype=np.float32)
    U = np.ascontiguousarray(U, dtype=np.float32)
    Y = np.empty_like(G)
    lib().oracle_glu(_p(G), _p(U), _p(Y), ctypes.c_long(G.size), act)
    return Y


def pack_q4(W, zero_scale=1.0):
    """W[OUT,IN] float32 -> (Wq uint8 [OUT,IN/2], sc float32 [OUT,IN/32]); RTN, scale = max|w|/7."""
    W = np.ascontiguousarray(W, dtype=np.float32)
    OUT, IN = W.shape
    Wq = np.empty((OUT, IN // 2), dtype=np.uint8)
    sc = np.empty((OUT, IN // QBLK), dtype=np.float32)
    lib().oracle_pack_q4(_p(W), OUT, IN, _p(Wq), _p(sc), ctypes.c_float(zero_scale))
    return Wq, sc


def _sd(sw):
    assert sw.dtype in (np.float32, np.float16)
    return 1 if sw.dtype == np.float16 else 0


def group_dots(xq, Wq):
    M, K = xq.shape
    N = Wq.shape[0]
    D = np.empty((M, N, K // QBLK), dtype=np.int32)
    lib().oracle_group_dots(_p(np.ascontiguousarray(xq)), _p(np.ascontiguousarray(Wq)), _p(D), M, N, K)
    return D


def _run(fn, out_dtype, xq, xs, Wq, sw, extra=()):
    M, K = xq.shape
    N = Wq.shape[0]
    Y = np.empty((M, N), dtype=out_dtype)
    fn(_p(np.ascontiguousarray(xq)), _p(np.ascontiguousarray(xs)), _p(np.ascontiguousarray(Wq)),
       _p(np.ascontiguousarray(sw)), _p(Y), M, N, K, _sd(sw), *extra)
    return Y


def w4a8_f64(xq, xs, Wq, sw):
    """fp64 golden of tests/test_w4a8.cu:44-56."""
    return _run(lib().oracle_w4a8_f64, np.float64, xq, xs, Wq, sw)


def gemv_w4a8(xq, xs, Wq, sw):
    """fp32 in the reference GEMV family's order (note the C signature is IN, OUT, S)."""
    M, K = xq.shape
    N = Wq.shape[0]
    Y = np.empty((M, N), dtype=np.float32)
    lib().oracle_gemv_w4a8(_p(np.ascontiguousarray(xq)), _p(np.ascontiguousarray(xs)), _p(np.ascontiguousarray(Wq)),
                           _p(np.ascontiguousarray(sw)), _p(Y), K, N, M, _sd(sw))
    return Y


def gemm_mmq_w4a8(xq, xs, Wq, sw):
    """fp32 in the reference MMQ / MMA family's order."""
    return _run(lib().oracle_gemm_mmq_w4a8, np.float32, xq, xs, Wq, sw)


def gemm_splitk_w4a8(xq, xs, Wq, sw, splitk):
    return _run(lib().oracle_gemm_splitk_w4a8, np.float32, xq, xs, Wq, sw, (int(splitk),))


def abs_terms(xq, xs, Wq, sw):
    return _run(lib().oracle_abs_terms, np.float64, xq, xs, Wq, sw)


def moe_w4a8(xq, xs, Wq, sw, idx, topk, x_per_slot, N, K):
    nslots = idx.shape[0]
    Y = np.empty((nslots, N), dtype=np.float32)
    lib().oracle_moe_w4a8(_p(np.ascontiguousarray(xq)), _p(np.ascontiguousarray(xs)), _p(np.ascontiguousarray(Wq)),
                          _p(np.ascontiguousarray(sw)), _p(np.ascontiguousarray(idx, dtype=np.int32)), _p(Y),
                          nslots, topk, int(x_per_slot), N, K, _sd(sw))
    return Y


def moe_combine(so, dw, topk):
    """out[b] = sum_k (ascending, from 0) dw[b*topk+k] * so[b*topk+k]; so [nslots, H] float32, dw [nslots] float32."""
    so = np.ascontiguousarray(so, dtype=np.float32)
    dw = np.ascontiguousarray(dw, dtype=np.float32)
    nslots, H = so.shape
    S = nslots // topk
    out = np.empty((S, H), dtype=np.float32)
    lib().oracle_moe_combine(_p(so), _p(dw), _p(out), S, topk, H)
    return out


def moe_block_w4a8(n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw, topk, act=0):
    """The routed-expert block in W4A8, stage by stage (models/moe_block.cuh:45-52 with the expert products in W4A8):
    quantize the tokens, gate|up product per slot against experts_gate_up[idx[slot]] ([E][2*MI][H], gate rows first,
    kernels/moe_fused.cuh:40-42), act(gate)*up, quantize, down product per slot against experts_down[idx[slot]]
    ([E][H][MI]), router weight and fixed-order combine (kernels/moe_fused.cuh:64,68-76).  Returns every stage."""
    n2 = np.ascontiguousarray(n2, dtype=np.float32)
    S, H = n2.shape
    E, MI2 = gu_wq.shape[0], gu_wq.shape[1]
    MI = MI2 // 2
    xq, xs, _ = quantize_x_q8(n2)
    gu = moe_w4a8(xq, xs, gu_wq.reshape(E * MI2, H // 2), gu_sc.reshape(E * MI2, H // QBLK), idx, topk, 0, MI2, H)
    hid = glu(gu[:, :MI], gu[:, MI:], act)
    xq_h, xs_h, _ = quantize_x_q8(hid)
    so = moe_w4a8(xq_h, xs_h, dn_wq.reshape(E * H, MI // 2), dn_sc.reshape(E * H, MI // QBLK), idx, topk, 1, H, MI)
    out = moe_combine(so, dw, topk)
    return {"xq": xq, "xs": xs, "gu": gu, "hid": hid, "xq_h": xq_h, "xs_h": xs_h, "so": so, "out": out}


def gemv_b200_order(xq, xs, Wq, sw):
    """fp32 in the B200 library's documented GEMV-family order (csrc/gemv_w4a8.cuh), for bit-exact checks."""
    M, K = xq.shape
    N = Wq.shape[0]
    Y = np.empty((M, N), dtype=np.float32)
    lib().oracle_gemv_b200_order(_p(np.ascontiguousarray(xq)), _p(np.ascontiguousarray(xs)),
                                 _p(np.ascontiguousarray(Wq)), _p(np.ascontiguousarray(sw)), _p(Y), K, N, M, _sd(sw))
    return Y


# ---- seeded synthetic inputs of the benchmark configurations' shapes ------------------------------------------------
def make_weights(N, K, seed, scale_dtype=0):
    """Packed int4 weights (every nibble uniform in 0..15, i.e. value uniform in [-8,7]) and group scales
    |N(0, 0.02)|/7, fp32 or fp16."""
    rng = np.random.default_rng(seed)
    Wq = rng.integers(0, 256, size=(N, K // 2), dtype=np.uint8)
    sw = (np.abs(rng.normal(0.0, 0.02, size=(N, K // QBLK))) / 7.0).astype(np.float32)
    if scale_dtype == 1:
        sw = sw.astype(np.float16)
    return Wq, sw


def make_activations(M, K, seed, outliers=False):
    """x ~ N(0,1) float32; with outliers=True a random 1 % of the entries is multiplied by 20."""
    rng = np.random.default_rng(seed)
    X = rng.normal(0.0, 1.0, size=(M, K)).astype(np.float32)
    if outliers:
        mask = rng.random(size=(M, K)) < 0.01
        X[mask] *= 20.0
    return X
