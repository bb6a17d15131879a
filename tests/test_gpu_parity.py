"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bars: quantized activations and int32 group dots bit-exact; fp32 outputs within
1e-5 relative.  The library's fp32 orders are fixed and restated in the oracle, so most fp32 checks here
are in fact bit-exact too: the GEMM family reproduces the reference MMQ order
(kernels/gemm_mmq.cuh:104-105) and so does the GEMV family's tensor-path kernel (S >= 2), the single-row dp4a GEMV
kernel has its own documented order; against the *other* order the
reference's own gate max|d|/rms < 1e-5 (tests/test_gemm_mmq.cu:28) applies.
Shapes follow the reference tests: tests/test_w4a8.cu:95-98, tests/test_gemm_mmq.cu:38,
tests/test_gemm_mma.cu:40, plus benchmark configuration 1 and ragged / partial-K-tile cases.
"""
import numpy as np
import pytest
import torch

from conftest import to_dev

pytestmark = pytest.mark.gpu
REL_TOL = 1e-5  # max|d| / rms(Y_ref), the reference's gate (tests/test_gemm_mmq.cu:28)


def rel_err(y, ref):
    ref = ref.astype(np.float64)
    rms = np.sqrt(np.mean(ref * ref))
    return float(np.max(np.abs(y.astype(np.float64) - ref)) / (rms if rms > 0 else 1.0))


def quantize_dev(w4a8, X_d):
    S, K = X_d.shape
    xq = torch.empty((S, K), dtype=torch.int8, device=X_d.device)
    xs = torch.empty((S, K // 32), dtype=torch.float32, device=X_d.device)
    xsum = torch.empty((S, K // 32), dtype=torch.int32, device=X_d.device)
    w4a8.launch_quantize_x_q8(X_d, xq, xs, xsum, K, S)
    return xq, xs, xsum


@pytest.mark.parametrize("S,K", [(1, 1024), (1, 3584), (5, 1024), (3, 32), (16, 5120), (37, 160), (513, 4096)])
def test_quantize_bit_exact(w4a8, oracle, cuda, S, K):
    X = oracle.make_activations(S, K, seed=100 + S + K, outliers=True)
    X[0, :32] = 0.0                      # an all-zero block: q = 0, d = 0 (kernels/quantize_x.cuh:35)
    if S > 1:
        X[1, 5] = 3.0e4                  # a dominant outlier
    xq_o, xs_o, xsum_o = oracle.quantize_x_q8(X)
    xq, xs, xsum = quantize_dev(w4a8, to_dev(X, cuda))
    torch.cuda.synchronize()
    assert np.array_equal(xq.cpu().numpy(), xq_o)
    assert np.array_equal(xs.cpu().numpy().view(np.uint32), xs_o.view(np.uint32))
    assert np.array_equal(xsum.cpu().numpy(), xsum_o)


def test_quantize_quotients_at_half_integers(w4a8, oracle, cuda):
    """Every element is built to land on, or within two ulp of, a half-integer quotient (k + 0.5) * d: the cases where
    q = rintf(x / d) (kernels/quantize_x.cuh:36) depends on the last bit of the IEEE division (a reciprocal multiply in its
    place was measured — no faster — and would have to fall back to the division exactly here)."""
    rng = np.random.default_rng(4242)
    S, K = 64, 2048
    X = np.empty((S, K), dtype=np.float32)
    for s_ in range(S):
        for b in range(K // 32):
            A = np.float32(rng.uniform(0.01, 300.0))
            d = np.float32(A / np.float32(127.0))
            blk = np.empty(32, dtype=np.float32)
            blk[0] = A
            for j in range(1, 32):
                x = np.float32(d * np.float32(rng.integers(0, 126) + 0.5))
                for _ in range(abs(j % 5 - 2)):
                    x = np.nextafter(x, np.float32(np.inf) if j % 5 > 2 else np.float32(0), dtype=np.float32)
                blk[j] = x if rng.random() < 0.5 else -x
            X[s_, b * 32:(b + 1) * 32] = blk
    xq_o, xs_o, xsum_o = oracle.quantize_x_q8(X)
    xq, xs, xsum = quantize_dev(w4a8, to_dev(X, cuda))
    torch.cuda.synchronize()
    assert np.array_equal(xq.cpu().numpy(), xq_o)
    assert np.array_equal(xs.cpu().numpy().view(np.uint32), xs_o.view(np.uint32)) and np.array_equal(xsum.cpu().numpy(), xsum_o)
    # the one-lane-per-element kernel (4-byte aligned input)
    buf = torch.zeros(S * K + 1, dtype=torch.float32, device=cuda)
    buf[1:] = to_dev(X, cuda).reshape(-1)
    xq2 = torch.empty((S, K), dtype=torch.int8, device=cuda)
    xs2 = torch.empty((S, K // 32), dtype=torch.float32, device=cuda)
    w4a8.launch_quantize_x_q8(buf.data_ptr() + 4, xq2, xs2, None, K, S)
    torch.cuda.synchronize()
    assert np.array_equal(xq2.cpu().numpy(), xq_o) and np.array_equal(xs2.cpu().numpy().view(np.uint32), xs_o.view(np.uint32))


def test_quantize_unaligned_and_null_xsum(w4a8, oracle, cuda):
    S, K = 3, 256
    X = oracle.make_activations(S, K, seed=7)
    xq_o, xs_o, _ = oracle.quantize_x_q8(X)
    buf = torch.zeros(S * K + 1, dtype=torch.float32, device=cuda)
    buf[1:] = to_dev(X, cuda).reshape(-1)            # 4-byte aligned only
    xq = torch.empty((S, K), dtype=torch.int8, device=cuda)
    xs = torch.empty((S, K // 32), dtype=torch.float32, device=cuda)
    w4a8.launch_quantize_x_q8(buf.data_ptr() + 4, xq, xs, None, K, S)
    torch.cuda.synchronize()
    assert np.array_equal(xq.cpu().numpy(), xq_o)
    assert np.array_equal(xs.cpu().numpy(), xs_o)


def make_case(oracle, M, N, K, seed, scale_dtype=0, outliers=False):
    X = oracle.make_activations(M, K, seed=seed, outliers=outliers)
    Wq, sw = oracle.make_weights(N, K, seed=seed + 1, scale_dtype=scale_dtype)
    xq, xs, _ = oracle.quantize_x_q8(X)
    return xq, xs, Wq, sw


@pytest.mark.parametrize("path", [0, 1, 2])
@pytest.mark.parametrize("M,N,K", [(1, 64, 256), (16, 8, 256), (5, 200, 160), (130, 140, 96), (200, 300, 1024)])
def test_group_dots_bit_exact(w4a8, oracle, cuda, path, M, N, K):
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=300 + M + N)
    D_o = oracle.group_dots(xq, Wq)
    D = torch.full((M, N, K // 32), 123456, dtype=torch.int32, device=cuda)
    w4a8.group_dots(to_dev(xq, cuda), to_dev(Wq, cuda), D, M, N, K, path=path)
    w4a8.device_status()
    assert np.array_equal(D.cpu().numpy(), D_o)


GEMV_SHAPES = [(1024, 256, 1), (1024, 2048, 1), (3584, 1024, 1), (1024, 4096, 5),   # tests/test_w4a8.cu:95-98
               (4096, 4096, 1),                                                     # benchmark configuration 1
               (160, 37, 3), (96, 9, 2), (5120, 1000, 16), (15360, 384, 8), (2048, 768, 7), (768, 2048, 12),
               (768, 2048, 1), (768, 1030, 1), (768, 3, 1)]                         # rows of 24 groups: the flat-group kernel, ragged last tile


def gemv_expected(oracle, xq, xs, Wq, sw, policy=0):
    """The documented fp32 order of w4a8_gemv.  A single row goes through the dp4a kernel or the bulk-copy stream, which
    share one chain order (auto picks by size and scale type; policy 3 forces the bulk-copy stream, 1 the dp4a kernel);
    the mma.sync tensor-path kernel (MMQ order, kernels/gemm_mmq.cuh:104-105) serves S >= 2, and S = 1 with fp16 scales
    when the bulk-copy stream does not take the row (K outside 2048..8192), when K % 256 == 0; the dp4a kernel everything
    else.  Policy 5 = the tcgen05 tensor path (MMQ order for every S) where K % 128 == 0 (K % 256 == 0 with fp16
    scales), else the dp4a kernel."""
    S, K = xq.shape
    fp16 = sw.dtype == np.float16
    if policy == 5:
        if K % (256 if fp16 else 128) == 0:
            return oracle.gemm_mmq_w4a8(xq, xs, Wq, sw)
        policy = 1
    bulk = S == 1 and K % (256 if fp16 else 128) == 0 and K <= 8192 and (policy == 3 or (policy == 0 and K >= 2048))
    mma = not bulk and K % 256 == 0 and (policy == 2 or (policy == 0 and (S >= 2 or fp16)))
    return oracle.gemm_mmq_w4a8(xq, xs, Wq, sw) if mma else oracle.gemv_b200_order(xq, xs, Wq, sw)


@pytest.mark.parametrize("policy", [0, 1, 2, 3, 5])
@pytest.mark.parametrize("scale_dtype", [0, 1])
@pytest.mark.parametrize("IN,OUT,S", GEMV_SHAPES)
def test_gemv_parity(w4a8, oracle, cuda, IN, OUT, S, scale_dtype, policy):
    if policy != 0 and scale_dtype == 1 and IN not in (1024, 5120, 768):
        pytest.skip("forced-kernel policies are covered on a subset of the fp16-scale shapes")
    xq, xs, Wq, sw = make_case(oracle, S, OUT, IN, seed=500 + IN + OUT + S, scale_dtype=scale_dtype)
    Y = torch.full((S + 1, OUT), float("nan"), dtype=torch.float32, device=cuda)          # last row: canary
    w4a8.config("gemv_kernel", policy)
    try:
        w4a8.launch_gemv_w4a8_sb(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq, cuda), to_dev(sw, cuda), Y, IN, OUT, S, scale_dtype)
        torch.cuda.synchronize()
    finally:
        w4a8.config("gemv_kernel", 0)
    y = Y.cpu().numpy()
    assert np.all(np.isnan(y[S])) and not np.any(np.isnan(y[:S]))
    y = y[:S]
    assert np.array_equal(y.view(np.uint32), gemv_expected(oracle, xq, xs, Wq, sw, policy).view(np.uint32))   # documented order
    assert rel_err(y, oracle.gemv_w4a8(xq, xs, Wq, sw)) < REL_TOL                                        # reference GEMV order
    assert np.max(np.abs(y - oracle.w4a8_f64(xq, xs, Wq, sw))) < 1e-2                                    # tests/test_w4a8.cu:83


def test_gemv_rows_independent_of_batch(w4a8, oracle, cuda):
    """A row's result does not depend on S or on its position (models/qwen35_batch.cu:270-273): for every S >= 2
    under the default policy, for every S >= 1 with the tensor-path kernel forced, and equal to the GEMM family."""
    IN, OUT, S = 2048, 520, 13
    xq, xs, Wq, sw = make_case(oracle, S, OUT, IN, seed=77)
    d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
    Y = torch.empty((S, OUT), dtype=torch.float32, device=cuda)
    w4a8.launch_gemv_w4a8_sb(d[0], d[1], d[2], d[3], Y, IN, OUT, S)
    for s in (0, 6, 11):                                   # pairs of rows, default policy
        y2 = torch.empty((2, OUT), dtype=torch.float32, device=cuda)
        w4a8.launch_gemm_batch_w4a8(d[0][s:s + 2].contiguous(), d[1][s:s + 2].contiguous(), d[2], d[3], y2, IN, OUT, 2)
        torch.cuda.synchronize()
        assert torch.equal(y2, Y[s:s + 2])
    w4a8.config("gemv_kernel", 2)
    try:
        for s in (0, 6, 12):                               # single rows, tensor-path kernel for every S
            y1 = torch.empty((1, OUT), dtype=torch.float32, device=cuda)
            w4a8.launch_gemv_w4a8(d[0][s:s + 1].contiguous(), d[1][s:s + 1].contiguous(), None, d[2], d[3], y1, IN, OUT, 1)
            torch.cuda.synchronize()
            assert torch.equal(y1[0], Y[s])
    finally:
        w4a8.config("gemv_kernel", 0)
    Yg = torch.empty((S, OUT), dtype=torch.float32, device=cuda)      # the GEMM family gives the same bits
    w4a8.launch_gemm_mmq_w4a8(d[0], d[1], d[2], d[3], Yg, S, OUT, IN)
    w4a8.device_status()
    assert torch.equal(Yg, Y)


GEMM_SHAPES = [(128, 128, 512), (256, 512, 1024), (200, 300, 256), (129, 140, 160),     # tests/test_gemm_mmq.cu:38
               (64, 128, 512), (129, 256, 1024),                                        # tests/test_gemm_mma.cu:40
               (17, 8, 32), (37, 3840, 3840), (513, 1000, 2048), (1, 5, 96)]


@pytest.mark.parametrize("scale_dtype", [0, 1])
@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_parity(w4a8, oracle, cuda, M, N, K, scale_dtype):
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=900 + M + N + K, scale_dtype=scale_dtype, outliers=True)
    Y = torch.full((M + 1, N), float("nan"), dtype=torch.float32, device=cuda)   # last row: canary
    w4a8.launch_gemm_mmq_w4a8(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq, cuda), to_dev(sw, cuda), Y, M, N, K, scale_dtype)
    w4a8.device_status()
    y = Y.cpu().numpy()
    assert np.all(np.isnan(y[M]))                                                       # nothing written past M rows
    y = y[:M]
    assert not np.any(np.isnan(y))
    assert np.array_equal(y.view(np.uint32), oracle.gemm_mmq_w4a8(xq, xs, Wq, sw).view(np.uint32))      # MMQ order, bitwise
    assert rel_err(y, oracle.gemv_w4a8(xq, xs, Wq, sw)) < REL_TOL                                        # tests/test_gemm_mmq.cu:28
    terms = oracle.abs_terms(xq, xs, Wq, sw)                                                             # tests/gemma4_mmq/shape.cu:105-117
    assert np.max(np.abs(y - oracle.w4a8_f64(xq, xs, Wq, sw)) / np.maximum(terms, 1e-30)) < REL_TOL


@pytest.mark.parametrize("scale_dtype", [0, 1])
@pytest.mark.parametrize("M,N,K", [(128, 128, 512), (200, 300, 256), (129, 140, 160), (17, 8, 32), (513, 1000, 2048), (1, 5, 96)])
def test_gemm_fp16_operand_kernel_same_bits(w4a8, oracle, cuda, M, N, K, scale_dtype):
    """config("gemm_kernel", 0) selects the fp16-operand tensor-core kernel: the same bits as the int8 one."""
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=1900 + M + N + K, scale_dtype=scale_dtype, outliers=True)
    d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
    want = oracle.gemm_mmq_w4a8(xq, xs, Wq, sw).view(np.uint32)
    try:
        for kernel in (0, 1):
            w4a8.config("gemm_kernel", kernel)
            Y = torch.full((M, N), float("nan"), dtype=torch.float32, device=cuda)
            w4a8.launch_gemm_mmq_w4a8(d[0], d[1], d[2], d[3], Y, M, N, K, scale_dtype)
            w4a8.device_status()
            assert np.array_equal(Y.cpu().numpy().view(np.uint32), want), kernel
    finally:
        w4a8.config("gemm_kernel", 1)


def test_gemm_deterministic_and_row_independent(w4a8, oracle, cuda):
    """30-run bitwise determinism (tests/test_gemm_mmq.cu:30-33); rows 7..13 of an M=14 run equal an M=7
    run of those rows (tools/probe_mmq_rowdep.cu)."""
    M, N, K = 300, 384, 1024
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=4242)
    d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
    Y0 = torch.empty((M, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemm_mmq_w4a8(d[0], d[1], d[2], d[3], Y0, M, N, K)
    for _ in range(30):
        Y = torch.empty((M, N), dtype=torch.float32, device=cuda)
        w4a8.launch_gemm_mmq_w4a8(d[0], d[1], d[2], d[3], Y, M, N, K)
        assert torch.equal(Y, Y0)
    Ya = torch.empty((14, N), dtype=torch.float32, device=cuda)
    Yb = torch.empty((7, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemm_mmq_w4a8(d[0][:14].contiguous(), d[1][:14].contiguous(), d[2], d[3], Ya, 14, N, K)
    w4a8.launch_gemm_mmq_w4a8(d[0][7:14].contiguous(), d[1][7:14].contiguous(), d[2], d[3], Yb, 7, N, K)
    w4a8.device_status()
    assert torch.equal(Ya[7:14], Yb)


@pytest.mark.parametrize("M,N,K,splitk", [(16, 256, 1024, 4), (14, 300, 2048, 0), (9, 128, 160, 3), (16, 128, 64, 8), (130, 140, 512, 2)])
def test_gemm_splitk(w4a8, oracle, cuda, M, N, K, splitk):
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=1300 + M + N + K)
    nbytes = w4a8.gemm_splitk_workspace_bytes(M, N, K, splitk)
    ws = torch.empty(max(nbytes, 16) // 4, dtype=torch.float32, device=cuda)
    Y = torch.empty((M, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemm_bm16_splitk(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq, cuda), to_dev(sw, cuda), Y, M, N, K,
                                 splitk=splitk, workspace=ws)
    w4a8.device_status()
    nsplit = nbytes // (M * N * 4) if nbytes else 1
    ref = oracle.gemm_splitk_w4a8(xq, xs, Wq, sw, nsplit)
    assert np.array_equal(Y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
    assert rel_err(Y.cpu().numpy(), oracle.gemm_mmq_w4a8(xq, xs, Wq, sw)) < REL_TOL


@pytest.mark.parametrize("tokens,topk,E,N,K,per_slot", [(8, 8, 128, 768, 2048, 0), (8, 8, 128, 2048, 768, 1), (3, 2, 4, 40, 96, 0)])
def test_moe_gemv(w4a8, oracle, cuda, tokens, topk, E, N, K, per_slot):
    rng = np.random.default_rng(99)
    idx = np.stack([rng.permutation(E)[:topk] for _ in range(tokens)]).astype(np.int32).reshape(-1)   # distinct per token
    nslots = tokens * topk
    rows = nslots if per_slot else tokens
    X = oracle.make_activations(rows, K, seed=5)
    Wq, sw = oracle.make_weights(E * N, K, seed=6)
    xq, xs, _ = oracle.quantize_x_q8(X)
    Y = torch.empty((nslots, N), dtype=torch.float32, device=cuda)
    w4a8.moe_gemv(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq, cuda), to_dev(sw, cuda), to_dev(idx, cuda), Y,
                  nslots, topk, per_slot, N, K, E)
    torch.cuda.synchronize()
    ref = oracle.moe_w4a8(xq, xs, Wq, sw, idx, topk, per_slot, N, K)
    assert rel_err(Y.cpu().numpy(), ref) < REL_TOL
    # bit-exact against the documented GEMV order applied per slot
    for slot in (0, nslots - 1):
        e, row = idx[slot], (slot if per_slot else slot // topk)
        r = oracle.gemv_b200_order(xq[row:row + 1], xs[row:row + 1], Wq[e * N:(e + 1) * N], sw[e * N:(e + 1) * N])
        assert np.array_equal(Y[slot].cpu().numpy().view(np.uint32), r[0].view(np.uint32))


def test_linear_dispatch_and_loader(w4a8, oracle, cuda, tmp_path):
    """mm(): quantize + GEMV for S <= 16, GEMM above; weights through the N-sharded loader (world 1 and 3)."""
    N, K = 300, 512
    Wq, sw = oracle.make_weights(N, K, seed=11)
    q4, sc = tmp_path / "w_q4.bin", tmp_path / "w_scale.bin"
    Wq.tofile(q4)
    sw.tofile(sc)
    whole = w4a8.load_qmat_shard(str(q4), str(sc), N, K, 0, 0, 1)
    assert (whole.row0, whole.rows) == (0, N)
    for S in (1, 16, 40):
        X = oracle.make_activations(S, K, seed=S)
        xq_o, xs_o, _ = oracle.quantize_x_q8(X)
        xq = torch.empty((S, K), dtype=torch.int8, device=cuda)
        xs = torch.empty((S, K // 32), dtype=torch.float32, device=cuda)
        xsum = torch.empty((S, K // 32), dtype=torch.int32, device=cuda)
        Y = torch.empty((S, N), dtype=torch.float32, device=cuda)
        w4a8.linear(to_dev(X, cuda), xq, xs, xsum, whole.wq, whole.sc, Y, S, N, K)
        w4a8.device_status()
        ref = gemv_expected(oracle, xq_o, xs_o, Wq, sw) if S <= 16 else oracle.gemm_mmq_w4a8(xq_o, xs_o, Wq, sw)
        assert np.array_equal(Y.cpu().numpy().view(np.uint32), ref.view(np.uint32))
        # the same product assembled from three row shards
        parts = []
        for r in range(3):
            m = w4a8.upload_qmat_shard(Wq, sw, N, K, 0, r, 3)
            Yr = torch.empty((S, m.rows), dtype=torch.float32, device=cuda)
            w4a8.linear(None, xq, xs, xsum, m.wq, m.sc, Yr, S, int(m.rows), K, skip_quantize=1)
            torch.cuda.synchronize()
            parts.append(Yr.cpu().numpy())
            w4a8.free_qmat(m)
        assert np.array_equal(np.concatenate(parts, axis=1).view(np.uint32), ref.view(np.uint32))
    w4a8.free_qmat(whole)
    with pytest.raises(w4a8.W4A8Error) as ei:
        w4a8.load_qmat_shard(str(q4), str(sc), N + 1, K, 0, 0, 1)      # file shorter than the shape: size mismatch
    assert ei.value.code == w4a8.ERR_IO


@pytest.mark.parametrize("pinned", [True, False])
@pytest.mark.parametrize("S,N,K", [(3, 200, 512), (1, 1000, 1024), (40, 7000, 1024)])
def test_linear_host_entry(w4a8, oracle, cuda, S, N, K, pinned):
    """mm() with host buffers: X in, quantize + product, Y out, synchronous.  Pinned buffers of a small step are read
    and written by the kernels themselves; pageable buffers, and steps above 1 MiB, go through the copy engines."""
    X = oracle.make_activations(S, K, seed=8)
    Wq, sw = oracle.make_weights(N, K, seed=9)
    Xh = torch.from_numpy(X)
    Yh = torch.full((S, N), float("nan"), dtype=torch.float32)
    if pinned:
        Xh, Yh = Xh.pin_memory(), Yh.pin_memory()
    Xd = torch.empty((S, K), dtype=torch.float32, device=cuda)
    xq = torch.empty((S, K), dtype=torch.int8, device=cuda)
    xs = torch.empty((S, K // 32), dtype=torch.float32, device=cuda)
    xsum = torch.empty((S, K // 32), dtype=torch.int32, device=cuda)
    Yd = torch.empty((S, N), dtype=torch.float32, device=cuda)
    w4a8.linear_host(Xh, Yh, Xd, xq, xs, xsum, Yd, to_dev(Wq, cuda), to_dev(sw, cuda), S, N, K)
    w4a8.device_status()
    xq_o, xs_o, _ = oracle.quantize_x_q8(X)
    want = gemv_expected(oracle, xq_o, xs_o, Wq, sw) if S <= 16 else oracle.gemm_mmq_w4a8(xq_o, xs_o, Wq, sw)
    assert np.array_equal(Yh.numpy().view(np.uint32), want.view(np.uint32))


# ---- benchmark configurations at their full shapes -----------------------------------------------------------------
@pytest.mark.parametrize("K,N", [(3840, 4096), (3840, 3840), (3840, 15360), (15360, 3840)])
def test_config3_gemma_layer_shapes_m8(w4a8, oracle, cuda, K, N):
    xq, xs, Wq, sw = make_case(oracle, 8, N, K, seed=K + N)
    Y = torch.empty((8, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemv_w4a8_sb(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq, cuda), to_dev(sw, cuda), Y, K, N, 8)
    torch.cuda.synchronize()
    assert np.array_equal(Y.cpu().numpy().view(np.uint32), gemv_expected(oracle, xq, xs, Wq, sw).view(np.uint32))


@pytest.mark.parametrize("M", [1, 2, 4, 8, 16])
def test_config2_decode_sweep_full_shape(w4a8, oracle, cuda, M):
    K, N = 5120, 17408
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=20260002 + M)
    Y = torch.empty((M, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemv_w4a8_sb(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq, cuda), to_dev(sw, cuda), Y, K, N, M)
    torch.cuda.synchronize()
    y = Y.cpu().numpy()
    assert np.array_equal(y.view(np.uint32), gemv_expected(oracle, xq, xs, Wq, sw).view(np.uint32))
    assert rel_err(y, oracle.w4a8_f64(xq, xs, Wq, sw)) < REL_TOL


@pytest.mark.parametrize("M", [512, 2048, 8192])
def test_config4_prefill_gemm_full_shape_sampled_rows(w4a8, oracle, cuda, M):
    """M = 512, 2048, 8192 (the reference bench's sizes, tools/bench_mmq_tune.cu:30), K=5120, N=17408 with 1 % outliers
    x20, quantize_x on the device.  The oracle cannot do the whole product in seconds, so: xq/xs/xsum of all rows exact;
    a sample of output rows bit-exact (rows are independent of M in the reference, tools/probe_mmq_rowdep.cu, so a row
    equals the M=1 product of that row); a second run bitwise equal."""
    K, N = 5120, 17408
    X = oracle.make_activations(M, K, seed=20260004, outliers=True)
    Wq, sw = oracle.make_weights(N, K, seed=20260005)
    xq_o, xs_o, xsum_o = oracle.quantize_x_q8(X)
    xq, xs, xsum = quantize_dev(w4a8, to_dev(X, cuda))
    torch.cuda.synchronize()
    assert np.array_equal(xq.cpu().numpy(), xq_o) and np.array_equal(xs.cpu().numpy(), xs_o) and np.array_equal(xsum.cpu().numpy(), xsum_o)
    Wq_d, sw_d = to_dev(Wq, cuda), to_dev(sw, cuda)
    Y = torch.empty((M, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemm_mmq_w4a8(xq, xs, Wq_d, sw_d, Y, M, N, K)
    w4a8.device_status()
    rows = np.unique(np.array([0, 1, 127, 128, 777 % M, M // 2 - 1, M // 2, M - 2, M - 1]))
    ref = oracle.gemm_mmq_w4a8(xq_o[rows], xs_o[rows], Wq, sw)
    assert np.array_equal(Y[torch.from_numpy(rows).to(cuda)].cpu().numpy().view(np.uint32), ref.view(np.uint32))
    Y2 = torch.empty((M, N), dtype=torch.float32, device=cuda)
    w4a8.launch_gemm_mmq_w4a8(xq, xs, Wq_d, sw_d, Y2, M, N, K)
    w4a8.device_status()
    assert torch.equal(Y, Y2)


def test_config5_moe_shapes(w4a8, oracle, cuda):
    """128 experts, top-8, gate/up K=2048 -> N=768 and down K=768 -> N=2048, 32 tokens (256 slots)."""
    E, topk, tokens = 128, 8, 32
    rng = np.random.default_rng(5)
    idx = np.stack([rng.permutation(E)[:topk] for _ in range(tokens)]).astype(np.int32).reshape(-1)
    for (K, N, per_slot) in [(2048, 768, 0), (768, 2048, 1)]:
        rows = tokens * topk if per_slot else tokens
        X = oracle.make_activations(rows, K, seed=K)
        Wq, sw = oracle.make_weights(E * N, K, seed=N)
        xq, xs, _ = oracle.quantize_x_q8(X)
        Y = torch.empty((tokens * topk, N), dtype=torch.float32, device=cuda)
        w4a8.moe_gemv(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq, cuda), to_dev(sw, cuda), to_dev(idx, cuda), Y,
                      tokens * topk, topk, per_slot, N, K, E)
        torch.cuda.synchronize()
        assert rel_err(Y.cpu().numpy(), oracle.moe_w4a8(xq, xs, Wq, sw, idx, topk, per_slot, N, K)) < REL_TOL


# ---- several matrices against one quantized input (gate + up, q + k + v) --------------------------------------
@pytest.mark.parametrize("scale_dtype", [0, 1])
@pytest.mark.parametrize("S,K,OUTS", [(1, 5120, (1000, 1000)), (1, 2048, (40, 3000, 7)), (1, 4096, (512, 256, 256, 77)),
                                      (1, 512, (100, 60)), (5, 2048, (300, 200)), (1, 5120, (17408,))])
def test_gemv_multi_equals_separate_calls(w4a8, oracle, cuda, S, K, OUTS, scale_dtype):
    """w4a8_gemv_multi (one launch on the bulk-copy kernel for a single row of 2048..8192 elements; else one call per
    matrix) gives each matrix the bits of its own w4a8_gemv call, and those are the documented order."""
    mats = [make_case(oracle, S, n, K, seed=4000 + n + i, scale_dtype=scale_dtype) for i, n in enumerate(OUTS)]
    xq, xs = mats[0][0], mats[0][1]
    xq_d, xs_d = to_dev(xq, cuda), to_dev(xs, cuda)
    Wq_d = [to_dev(m[2], cuda) for m in mats]
    sw_d = [to_dev(m[3], cuda) for m in mats]
    Ys = [torch.full((S + 1, n), float("nan"), dtype=torch.float32, device=cuda) for n in OUTS]     # last row: canary
    w4a8.gemv_multi(xq_d, xs_d, Wq_d, sw_d, Ys, OUTS, K, S, scale_dtype)
    w4a8.device_status()
    for i, n in enumerate(OUTS):
        Y1 = torch.empty((S, n), dtype=torch.float32, device=cuda)
        w4a8.launch_gemv_w4a8_sb(xq_d, xs_d, Wq_d[i], sw_d[i], Y1, K, n, S, scale_dtype)
        torch.cuda.synchronize()
        y = Ys[i].cpu().numpy()
        assert np.all(np.isnan(y[S]))
        assert np.array_equal(y[:S].view(np.uint32), Y1.cpu().numpy().view(np.uint32))
        assert np.array_equal(y[:S].view(np.uint32), gemv_expected(oracle, xq, xs, mats[i][2], mats[i][3]).view(np.uint32))
