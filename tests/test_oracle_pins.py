"""CPU tests that PIN the oracle (oracle/w4a8_oracle.c) to the reference:

  - golden byte fixtures produced by importing the reference's own tools/extract_weights.py and
    tools/qat_golden_loader.py (tests/golden/*.npz, generator committed beside them);
  - the reference unit tests' LCG-seeded cases, regenerated from their seeds with their gates applied
    (tests/test_w4a8.cu:16,36-56,75-98; tests/test_mma_b1.cu:40-65);
  - an independent numpy restatement of the quantizer and the integer dots;
  - the frozen on-disk format checks of tests/test_quantization_variants.py:20-34 and
    tests/test_qat_golden.py:13-30.
(On a GPU box tests/test_gpu_vs_reference.py additionally checks the oracle bit-for-bit against the
reference's own CUDA kernels.)
"""
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def unpack_ref(packed, scale):
    """Decode exactly as tests/test_quantization_variants.py:13-17 does."""
    v = np.empty(packed.size * 2, dtype=np.float32)
    v[::2] = packed & 15
    v[1::2] = packed >> 4
    return (v.reshape(-1, 32) - 8) * scale[:, None]


def np_quantize(X):
    """Independent numpy statement of kernels/quantize_x.cuh:31-38."""
    S, K = X.shape
    blk = X.reshape(S, K // 32, 32)
    amax = np.abs(blk).max(axis=2)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(amax[..., None] == 0, 0, np.rint((blk / d[..., None]).astype(np.float32)))
    q = np.clip(q, -127, 127).astype(np.int32)
    return q.reshape(S, K).astype(np.int8), d, q.sum(axis=2).astype(np.int32)


def np_weights(Wq):
    N, K2 = Wq.shape
    w = np.empty((N, K2 * 2), dtype=np.int32)
    w[:, 0::2] = Wq & 15
    w[:, 1::2] = Wq >> 4
    return w - 8


def test_pack_matches_reference_extract_weights_fixture(oracle):
    g = np.load(os.path.join(GOLD, "rtn_q4.npz"))
    Wq, sc = oracle.pack_q4(g["w"], zero_scale=1e-8)
    assert Wq.reshape(-1).tobytes() == g["packed"].tobytes()
    assert sc.reshape(-1).tobytes() == g["scale"].tobytes()
    assert g["scale"][0] == np.float32(1e-8) and np.all(g["packed"][:16] == 0x88)   # the all-zero block


def test_weight_decode_matches_reference_loader_fixture(oracle):
    g = np.load(os.path.join(GOLD, "dequant.npz"))
    packed, scale = g["packed"], g["scale"]
    K = 160
    Wq = packed.reshape(-1, K // 2)
    N = Wq.shape[0]
    # x = one-hot rows with xs = 1 turn the oracle's product into a dequantiser: Y[k, n] = w(n,k) * scale
    xq = np.zeros((K, K), dtype=np.int8)
    xq[np.arange(K), np.arange(K)] = 1
    xs = np.ones((K, K // 32), dtype=np.float32)
    for key, sw in (("dequant_fp32_scale", scale.reshape(N, -1)), ("dequant_fp16_scale", scale.astype(np.float16).reshape(N, -1))):
        Y = oracle.gemm_mmq_w4a8(xq, xs, Wq, sw)
        assert np.array_equal(Y.T.reshape(-1), g[key]), key
        assert np.array_equal(oracle.gemv_w4a8(xq, xs, Wq, sw).T.reshape(-1), g[key])


def test_frozen_rtn_formula_and_nibble_order(oracle):
    # tests/test_quantization_variants.py:20-34
    w = np.random.default_rng(31).normal(size=(5, 64)).astype(np.float32)
    w[0, :32] = 0
    block = w.reshape(-1, 32)
    scale = np.max(np.abs(block), axis=1) / 7
    scale[scale == 0] = 1e-8
    q = np.clip(np.round(block / scale[:, None]) + 8, 0, 15).astype(np.uint8).ravel()
    expected = q[::2] | (q[1::2] << 4)
    Wq, sc = oracle.pack_q4(w, zero_scale=1e-8)
    assert Wq.reshape(-1).tobytes() == expected.tobytes()
    assert sc.reshape(-1).tobytes() == scale.astype(np.float32).tobytes()
    # tests/test_qat_golden.py:13-22: bytes 0..15 with scale 0.125 decode to (low-8)*0.125, -1
    packed = np.arange(16, dtype=np.uint8)
    exp = np.array([v for low in range(16) for v in ((low - 8) * 0.125, -1)], dtype=np.float32)
    assert np.array_equal(unpack_ref(packed, np.array([0.125], dtype=np.float32)).ravel(), exp)
    assert np.array_equal(np_weights(packed.reshape(1, 16)).ravel() * np.float32(0.125), exp)


def test_quantizer_against_numpy_restatement(oracle):
    for S, K, seed in [(1, 1024, 1), (5, 1024, 2), (16, 5120, 3), (37, 160, 4)]:
        X = oracle.make_activations(S, K, seed=seed, outliers=True)
        X[0, :32] = 0
        xq, xs, xsum = oracle.quantize_x_q8(X)
        q2, d2, s2 = np_quantize(X)
        assert np.array_equal(xq, q2) and np.array_equal(xs.view(np.uint32), d2.view(np.uint32)) and np.array_equal(xsum, s2)
        assert xs[0, 0] == 0 and not xq[0, :32].any()
        assert np.abs(xq.astype(np.int32)).max() <= 127


@pytest.mark.parametrize("IN,OUT,S", [(1024, 256, 1), (1024, 2048, 1), (3584, 1024, 1), (1024, 4096, 5)])
def test_reference_test_w4a8_cases(oracle, IN, OUT, S):
    """tests/test_w4a8.cu: LCG seed 12345 carried across its four run() calls; gates xq/xsum exact, |Y-gold|<1e-2."""
    seed = 12345
    for (i_, o_, s_) in [(1024, 256, 1), (1024, 2048, 1), (3584, 1024, 1), (1024, 4096, 5)]:
        X, seed = oracle.lcg_fill(s_ * i_, 2.0, seed)
        W, seed = oracle.lcg_fill(o_ * i_, 0.5, seed)
        if (i_, o_, s_) == (IN, OUT, S):
            break
    X, W = X.reshape(S, IN), W.reshape(OUT, IN)
    Wq, sc = oracle.pack_q4(W, zero_scale=1.0)
    xq, xs, xsum = oracle.quantize_x_q8(X)
    q2, d2, s2 = np_quantize(X)                              # the test's host quantizer (:36-43), restated
    assert np.array_equal(xq, q2) and np.array_equal(xsum, s2)
    gold = oracle.w4a8_f64(xq, xs, Wq, sc)
    wv = np_weights(Wq).astype(np.float64) * np.repeat(sc.astype(np.float64), 32, axis=1)     # :44-56 in numpy
    xv = xq.astype(np.float64) * np.repeat(xs.astype(np.float64), 32, axis=1)
    assert np.max(np.abs(gold - xv @ wv.T)) < 1e-9
    for y in (oracle.gemv_w4a8(xq, xs, Wq, sc), oracle.gemm_mmq_w4a8(xq, xs, Wq, sc), oracle.gemv_b200_order(xq, xs, Wq, sc)):
        assert np.max(np.abs(y - gold)) < 1e-2               # tests/test_w4a8.cu:83


def test_reference_test_mma_b1_case(oracle):
    """tests/test_mma_b1.cu:40-65: M=16, N=8, K=256, LCG seed 7; gate max err / rms < 1e-5 against sum_b dot*xs*sw."""
    M, N, K = 16, 8, 256
    Xf, seed = oracle.lcg_fill(M * K, 1.0, 7)
    Wf, seed = oracle.lcg_fill(N * K, 0.3, seed)
    Wq, sw = oracle.pack_q4(Wf.reshape(N, K), zero_scale=1.0)
    xq, xs, _ = oracle.quantize_x_q8(Xf.reshape(M, K))
    D = oracle.group_dots(xq, Wq)
    assert np.array_equal(D, np.einsum("mbk,nbk->mnb", xq.reshape(M, -1, 32).astype(np.int64),
                                       np_weights(Wq).reshape(N, -1, 32).astype(np.int64)).astype(np.int32))
    ref = (D.astype(np.float64) * xs[:, None, :].astype(np.float64) * sw[None].astype(np.float64)).sum(-1)
    rms = np.sqrt(np.mean(ref * ref))
    for y in (oracle.gemm_mmq_w4a8(xq, xs, Wq, sw), oracle.gemv_w4a8(xq, xs, Wq, sw)):
        assert np.max(np.abs(y - ref)) / rms < 1e-5


def test_orders_and_splitk_and_fp16_scales(oracle):
    M, N, K = 7, 50, 2048
    X = oracle.make_activations(M, K, seed=9)
    xq, xs, _ = oracle.quantize_x_q8(X)
    for sd in (0, 1):
        Wq, sw = oracle.make_weights(N, K, seed=10, scale_dtype=sd)
        gold = oracle.w4a8_f64(xq, xs, Wq, sw)
        rms = np.sqrt(np.mean(gold * gold))
        assert np.array_equal(oracle.gemm_splitk_w4a8(xq, xs, Wq, sw, 1).view(np.uint32), oracle.gemm_mmq_w4a8(xq, xs, Wq, sw).view(np.uint32))
        for y in (oracle.gemv_w4a8(xq, xs, Wq, sw), oracle.gemm_mmq_w4a8(xq, xs, Wq, sw), oracle.gemm_splitk_w4a8(xq, xs, Wq, sw, 4),
                  oracle.gemv_b200_order(xq, xs, Wq, sw)):
            assert np.max(np.abs(y - gold)) / rms < 1e-5
        if sd == 1:   # fp16 scales are read as their exact float value (kernels/qscale.cuh:6)
            assert np.array_equal(oracle.gemm_mmq_w4a8(xq, xs, Wq, sw), oracle.gemm_mmq_w4a8(xq, xs, Wq, sw.astype(np.float32)))
    # integer dots stay inside +-32512 and within 24 bits, so (float)D is exact
    D = oracle.group_dots(xq, Wq)
    assert np.abs(D).max() <= 127 * 8 * 32


def test_moe_oracle_is_dense_product_per_expert(oracle):
    E, N, K, tokens, topk = 6, 24, 96, 3, 2
    Wq, sw = oracle.make_weights(E * N, K, seed=3)
    X = oracle.make_activations(tokens, K, seed=4)
    xq, xs, _ = oracle.quantize_x_q8(X)
    idx = np.array([0, 5, 2, 2, 4, 1], dtype=np.int32)
    Y = oracle.moe_w4a8(xq, xs, Wq, sw, idx, topk, 0, N, K)
    for slot, e in enumerate(idx):
        t = slot // topk
        ref = oracle.gemm_mmq_w4a8(xq[t:t + 1], xs[t:t + 1], Wq[e * N:(e + 1) * N], sw[e * N:(e + 1) * N])
        assert np.array_equal(Y[slot], ref[0])


def test_oracle_rmsnorm_and_glu_against_float64(oracle):
    """The producers restated for the fused quantize entries: the reference's formulas (kernels/rmsnorm.cuh:5,28,50,
    kernels/swiglu.cuh:4,17) evaluated in float64 agree with the fp32 restatement to fp32 rounding."""
    rng = np.random.default_rng(3)
    X = rng.normal(0, 2, size=(4, 5120)).astype(np.float32)
    W = rng.normal(0, 0.3, size=5120).astype(np.float32)
    x64 = X.astype(np.float64)
    inv = 1.0 / np.sqrt(np.mean(x64 * x64, axis=1, keepdims=True) + 1e-6)
    for variant, want in ((0, x64 * inv * W), (1, x64 * inv * (1.0 + W.astype(np.float64))), (2, x64 * inv)):
        got = oracle.rmsnorm(X, W, 1e-6, variant)
        assert np.max(np.abs(got - want) / (np.abs(want) + 1e-6)) < 2e-6
    G = rng.normal(0, 2, size=(3, 768)).astype(np.float32)
    U = rng.normal(0, 1, size=(3, 768)).astype(np.float32)
    g64, u64 = G.astype(np.float64), U.astype(np.float64)
    silu = g64 / (1.0 + np.exp(-g64)) * u64
    gelu = 0.5 * g64 * (1.0 + np.tanh(0.7978845608028654 * (g64 + 0.044715 * g64 ** 3))) * u64
    assert np.max(np.abs(oracle.glu(G, U, 0) - silu)) < 2e-6 * np.max(np.abs(silu))
    assert np.max(np.abs(oracle.glu(G, U, 1) - gelu)) < 2e-6 * np.max(np.abs(gelu))
