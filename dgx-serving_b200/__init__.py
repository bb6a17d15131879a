"""Host-side Python binding of libw4a8_b200.so, the B200 (sm_100a) W4A8 quantized-matmul library.

The product is the C-ABI shared library (include/w4a8_b200.h) plus the C++ shim launchers in
kernels/*.cuh that carry the reference's launcher names.  This module is the thin ctypes layer the
tests and the benchmark use to call that ABI with torch tensors as device memory; torch is plumbing
(allocation, streams, torch.distributed), never a compute path.  There is no CPU or torch fallback:
if the library is missing or the device is not sm_100 every call raises.

Function names and argument order mirror the reference launchers
(kernels/quantize_x.cuh:41, kernels/gemv_w4a8.cuh:155,168, kernels/gemm_batch.cuh:228,
kernels/gemm_mmq.cuh:230, kernels/gemm_mmq_raster.cuh:115).
"""
import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("W4A8_LIB") or os.path.join(_HERE, "libw4a8_b200.so")   # W4A8_LIB: another build, for A/B timing
QBLK = 32

OK, ERR_ARG, ERR_ALIGN, ERR_CUDA, ERR_IO, ERR_DEVICE, ERR_UNSUPPORTED, ERR_WORKSPACE = range(8)

_lib = None


class W4A8Error(RuntimeError):
    def __init__(self, code, text):
        super().__init__("w4a8 error %d: %s" % (code, text))
        self.code = code


class QMat(ctypes.Structure):
    """Mirror of w4a8_qmat (the N-sharded form of the reference's QMat, runtime/weights_qwen.h:8)."""
    _fields_ = [("wq", ctypes.c_void_p), ("sc", ctypes.c_void_p), ("row0", ctypes.c_int64),
                ("rows", ctypes.c_int64), ("N", ctypes.c_int64), ("K", ctypes.c_int64),
                ("scale_dtype", ctypes.c_int)]


class MoeLayout(ctypes.Structure):
    """Mirror of w4a8_moe_layout: byte offsets of the routed-expert block's intermediates in the caller's workspace."""
    _fields_ = [(n, ctypes.c_size_t) for n in ("perm", "pos", "offsets", "items", "num_items", "xq", "xs", "xq_g", "xs_g", "gu",
                                               "xq_h", "xs_h", "sout", "bytes")]


_P, _I, _Z, _L = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_int64
_SIGNATURES = {
    "w4a8_version": (_I, []),
    "w4a8_last_error": (ctypes.c_char_p, []),
    "w4a8_device_status": (_I, [ctypes.POINTER(ctypes.c_uint32)]),
    "w4a8_config": (_I, [ctypes.c_char_p, _I]),
    "w4a8_quantize_x_q8": (_I, [_P, _P, _P, _P, _I, _I, _P]),
    "w4a8_rmsnorm_quantize_x_q8": (_I, [_P, _P, ctypes.c_float, _I, _P, _P, _P, _P, _I, _I, _P]),
    "w4a8_glu_quantize_x_q8": (_I, [_P, _P, _I, _P, _P, _P, _P, _I, _I, _P]),
    "w4a8_gemv": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "w4a8_gemv_multi": (_I, [_P, _P, _I, _P, _P, _P, _P, _I, _I, _I, _P]),
    "w4a8_gemm": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "w4a8_gemm_splitk_workspace_bytes": (_Z, [_I, _I, _I, _I]),
    "w4a8_gemm_splitk": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "w4a8_gemm_splitk_static": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "w4a8_group_dots": (_I, [_P, _P, _P, _I, _I, _I, _I, _P]),
    "w4a8_linear": (_I, [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _P]),
    "w4a8_linear_host": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P]),
    "w4a8_moe_gemv": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P]),
    "w4a8_moe_layout_for": (_I, [_I, _I, _I, _I, _I, ctypes.POINTER(MoeLayout)]),
    "w4a8_moe_block": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "w4a8_moe_block_shard": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _Z, _P, _Z, ctypes.c_uint32, _I, _I, _P]),
    "w4a8_shard_rows": (_I, [_L, _I, _I, ctypes.POINTER(_L), ctypes.POINTER(_L)]),
    "w4a8_load_qmat_shard": (_I, [ctypes.c_char_p, ctypes.c_char_p, _L, _L, _I, _I, _I, ctypes.POINTER(QMat)]),
    "w4a8_upload_qmat_shard": (_I, [_P, _P, _L, _L, _I, _I, _I, ctypes.POINTER(QMat)]),
    "w4a8_free_qmat": (_I, [ctypes.POINTER(QMat)]),
    "w4a8_arena_create": (_I, [_Z, _I, _I, ctypes.POINTER(_P)]),
    "w4a8_arena_base": (_P, [_P]),
    "w4a8_arena_connect": (_I, [_P, ctypes.POINTER(_P)]),
    "w4a8_arena_destroy": (_I, [_P]),
    "w4a8_ipc_export": (_I, [_P, ctypes.c_char_p]),
    "w4a8_ipc_open": (_I, [ctypes.c_char_p, ctypes.POINTER(_P)]),
    "w4a8_ipc_close": (_I, [_P]),
    "w4a8_gemv_allgather": (_I, [_P, _P, _P, _P, _P, _Z, _I, _I, _I, _I, _I, _I, ctypes.c_uint32, _P]),
    "w4a8_gemm_allgather": (_I, [_P, _P, _P, _P, _P, _Z, _I, _I, _I, _I, _I, _I, ctypes.c_uint32, _P]),
    "w4a8_allgather_wait": (_I, [_P, ctypes.c_uint32, _I, _P]),
    "w4a8_gemv_allgather_sync": (_I, [_P, _P, _P, _P, _P, _Z, _I, _I, _I, _I, _I, _I, ctypes.c_uint32, _I, _P]),
    "w4a8_gemm_allgather_sync": (_I, [_P, _P, _P, _P, _P, _Z, _I, _I, _I, _I, _I, _I, ctypes.c_uint32, _I, _P]),
    "w4a8_arena_advance_epoch": (_I, [_P, ctypes.c_uint32, _P]),
}
EXPORTS = tuple(_SIGNATURES)


def lib():
    """Loads the C-ABI library (once).  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError("%s not built; run python dgx-serving_b200/build.py (needs nvcc). "
                               "This library has no CPU or PyTorch fallback." % LIB_PATH)
        l = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.restype, fn.argtypes = res, args
        _lib = l
    return _lib


def _check(rc):
    if rc != OK:
        raise W4A8Error(rc, lib().w4a8_last_error().decode())


def _ptr(t):
    if t is None:
        return None
    if isinstance(t, int):
        return t
    return t.data_ptr()


def _stream(stream):
    if stream is None:
        import torch
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def config(key, value):
    """Run-time policy switch, e.g. config("gemv_kernel", 2): tensor-path GEMV for every S (see include/w4a8_b200.h)."""
    _check(lib().w4a8_config(key.encode(), int(value)))


def device_status():
    """Synchronises and raises if a kernel recorded a device-side error (a bounded wait ran out)."""
    d = ctypes.c_uint32(0)
    _check(lib().w4a8_device_status(ctypes.byref(d)))


def launch_quantize_x_q8(X, xq, xs, xsum, IN, S, stream=None):
    _check(lib().w4a8_quantize_x_q8(_ptr(X), _ptr(xq), _ptr(xs), _ptr(xsum), IN, S, _stream(stream)))


def launch_rmsnorm_quantize_x_q8(X, W, eps, variant, Y, xq, xs, xsum, IN, S, stream=None):
    """RMSNorm (variant 0: * W, 1: * (1 + W), 2: no scale) and quantize_x in one kernel; Y (may be None) also gets the
    fp32 intermediate.  Same bits as the reference's launch_rmsnorm* followed by launch_quantize_x_q8."""
    _check(lib().w4a8_rmsnorm_quantize_x_q8(_ptr(X), _ptr(W), float(eps), variant, _ptr(Y), _ptr(xq), _ptr(xs), _ptr(xsum), IN, S,
                                            _stream(stream)))


def launch_glu_quantize_x_q8(G, U, act, Y, xq, xs, xsum, IN, S, stream=None):
    """SwiGLU (act 0) or GeGLU (act 1) of (G, U) and quantize_x in one kernel; Y (may be None) also gets the fp32 product."""
    _check(lib().w4a8_glu_quantize_x_q8(_ptr(G), _ptr(U), act, _ptr(Y), _ptr(xq), _ptr(xs), _ptr(xsum), IN, S, _stream(stream)))


def gemv_multi(xq, xs, Wqs, sws, Ys, OUTs, IN, S, scale_dtype=0, stream=None):
    """Several matrices (at most 4) against the same activation rows in one call; one launch for a single row on the
    bulk-copy kernel.  Each Ys[i] equals launch_gemv_w4a8 of matrix i."""
    n = len(Wqs)
    arr = lambda xs_: (ctypes.c_void_p * n)(*[_ptr(t) for t in xs_])
    outs = (ctypes.c_int * n)(*[int(o) for o in OUTs])
    _check(lib().w4a8_gemv_multi(_ptr(xq), _ptr(xs), n, arr(Wqs), arr(sws), arr(Ys), outs, IN, S, scale_dtype, _stream(stream)))


def launch_gemv_w4a8(xq, xs, xsum, Wq, sw, Y, IN, OUT, S, scale_dtype=0, stream=None):
    """xsum is accepted and ignored, as in the reference (kernels/gemv_w4a8.cuh:23-25)."""
    _check(lib().w4a8_gemv(_ptr(xq), _ptr(xs), _ptr(Wq), _ptr(sw), _ptr(Y), IN, OUT, S, scale_dtype, _stream(stream)))


def launch_gemv_w4a8_sb(xq, xs, Wq, sw, Y, IN, OUT, S, scale_dtype=0, stream=None):
    _check(lib().w4a8_gemv(_ptr(xq), _ptr(xs), _ptr(Wq), _ptr(sw), _ptr(Y), IN, OUT, S, scale_dtype, _stream(stream)))


launch_gemv_w4a8_mlp = launch_gemv_w4a8_mlp_auto = launch_gemv_w4a8_g4 = launch_gemv_w4a8
launch_gemv_w4a8_sb_g4 = launch_gemv_w4a8_sb


def launch_gemm_batch_w4a8(xq, xs, Wq, sw, Y, IN, OUT, B, scale_dtype=0, stream=None):
    _check(lib().w4a8_gemv(_ptr(xq), _ptr(xs), _ptr(Wq), _ptr(sw), _ptr(Y), IN, OUT, B, scale_dtype, _stream(stream)))


def launch_gemm_mmq_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype=0, stream=None):
    _check(lib().w4a8_gemm(_ptr(X), _ptr(xs), _ptr(Wq), _ptr(sw), _ptr(Y), M, N, K, scale_dtype, _stream(stream)))


launch_gemm_mmq_w4a8_auto = launch_gemm_mma_w4a8 = launch_gemm_mmq_w4a8


def launch_gemm_mmq_raster_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype, raster, group, stream=None):
    """raster/group only re-order tiles in the reference (kernels/gemm_mmq_raster.cuh:16-27); results are equal."""
    launch_gemm_mmq_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype, stream)


def gemm_splitk_workspace_bytes(M, N, K, splitk=0):
    return int(lib().w4a8_gemm_splitk_workspace_bytes(M, N, K, splitk))


def launch_gemm_bm16_splitk(X, xs, Wq, sw, Y, M, N, K, scale_dtype=0, splitk=0, workspace=None, stream=None):
    nbytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    _check(lib().w4a8_gemm_splitk(_ptr(X), _ptr(xs), _ptr(Wq), _ptr(sw), _ptr(Y), M, N, K, scale_dtype, splitk,
                                  _ptr(workspace), nbytes, _stream(stream)))


SPLITK_STATIC_BYTES = 16 * 1024 * 1024


def launch_gemm_splitk_static(X, xs, Wq, sw, Y, M, N, K, scale_dtype=0, splitk=0, stream=None):
    """Split-K GEMM whose partial sums live in a buffer built into the library: no workspace, no allocation.
    For callers that cannot allocate at the point of the call; at most SPLITK_STATIC_BYTES of partial sums."""
    _check(lib().w4a8_gemm_splitk_static(_ptr(X), _ptr(xs), _ptr(Wq), _ptr(sw), _ptr(Y), M, N, K, scale_dtype, splitk,
                                         _stream(stream)))


def group_dots(xq, Wq, D, M, N, K, path=0, stream=None):
    _check(lib().w4a8_group_dots(_ptr(xq), _ptr(Wq), _ptr(D), M, N, K, path, _stream(stream)))


def linear(X, xq, xs, xsum, Wq, sw, Y, S, N, K, scale_dtype=0, skip_quantize=0, stream=None):
    """The mm() dispatcher of the model graphs (models/qwen35_decode.cu:51-62)."""
    _check(lib().w4a8_linear(_ptr(X), _ptr(xq), _ptr(xs), _ptr(xsum), _ptr(Wq), _ptr(sw), _ptr(Y), S, N, K,
                             scale_dtype, skip_quantize, _stream(stream)))


def linear_host(X_host, Y_host, X_dev, xq, xs, xsum, Y_dev, Wq, sw, S, N, K, scale_dtype=0, stream=None):
    """mm() with host activations in and host results out (pinned torch tensors or raw host pointers); synchronous."""
    _check(lib().w4a8_linear_host(_ptr(X_host), _ptr(Y_host), _ptr(X_dev), _ptr(xq), _ptr(xs), _ptr(xsum), _ptr(Y_dev), _ptr(Wq),
                                  _ptr(sw), S, N, K, scale_dtype, _stream(stream)))


def moe_gemv(xq, xs, Wq, sw, idx, Y, nslots, topk, x_per_slot, N, K, num_experts, scale_dtype=0, stream=None):
    _check(lib().w4a8_moe_gemv(_ptr(xq), _ptr(xs), _ptr(Wq), _ptr(sw), _ptr(idx), _ptr(Y), nslots, topk, x_per_slot,
                               N, K, num_experts, scale_dtype, _stream(stream)))


def moe_layout_for(S, topk, H, MI, experts):
    l = MoeLayout()
    _check(lib().w4a8_moe_layout_for(S, topk, H, MI, experts, ctypes.byref(l)))
    return l


def moe_block(n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw, out, S, topk, H, MI, num_experts, workspace, scale_dtype=0, act=0, stream=None):
    """The routed-expert block of models/moe_block.cuh:45-52 in W4A8 (w4a8_moe_block); workspace = a uint8 device tensor
    of moe_layout_for(...).bytes bytes."""
    _check(lib().w4a8_moe_block(_ptr(n2), _ptr(gu_wq), _ptr(gu_sc), _ptr(dn_wq), _ptr(dn_sc), _ptr(idx), _ptr(dw), _ptr(out), S, topk, H, MI,
                                num_experts, scale_dtype, act, _ptr(workspace), workspace.numel() * workspace.element_size(), _stream(stream)))


def moe_block_shard(n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw, out, S, topk, H, MI, expert_base, experts_local, workspace, arena, sout_offset,
                    epoch, scale_dtype=0, act=0, timeout_us=1000000, phase=0, stream=None):
    """Expert-sharded routed-expert block (w4a8_moe_block_shard): this rank's experts only, down outputs exchanged through the arenas."""
    _check(lib().w4a8_moe_block_shard(_ptr(n2), _ptr(gu_wq), _ptr(gu_sc), _ptr(dn_wq), _ptr(dn_sc), _ptr(idx), _ptr(dw), _ptr(out), S, topk, H, MI,
                                      expert_base, experts_local, scale_dtype, act, _ptr(workspace),
                                      workspace.numel() * workspace.element_size(), arena.handle, sout_offset, epoch, timeout_us, phase, _stream(stream)))


def shard_rows(N, rank, world):
    r0, rows = _L(0), _L(0)
    _check(lib().w4a8_shard_rows(N, rank, world, ctypes.byref(r0), ctypes.byref(rows)))
    return r0.value, rows.value


def load_qmat_shard(q4_path, scale_path, N, K, scale_dtype, rank, world):
    m = QMat()
    _check(lib().w4a8_load_qmat_shard(os.fsencode(q4_path), os.fsencode(scale_path), N, K, scale_dtype, rank, world,
                                      ctypes.byref(m)))
    return m


def upload_qmat_shard(host_wq, host_sc, N, K, scale_dtype, rank, world):
    """host_wq / host_sc: numpy arrays (or anything with .ctypes) holding the full [N] tensors."""
    m = QMat()
    _check(lib().w4a8_upload_qmat_shard(host_wq.ctypes.data, host_sc.ctypes.data, N, K, scale_dtype, rank, world,
                                        ctypes.byref(m)))
    return m


def free_qmat(m):
    _check(lib().w4a8_free_qmat(ctypes.byref(m)))


class Arena:
    """Peer-visible device memory for the fused GEMV + all-gather (w4a8_arena in include/w4a8_b200.h)."""

    def __init__(self, nbytes, rank, world):
        h = _P()
        _check(lib().w4a8_arena_create(nbytes, rank, world, ctypes.byref(h)))
        self.handle, self.rank, self.world, self.nbytes = h, rank, world, nbytes
        self.base = lib().w4a8_arena_base(h)
        self._opened = []

    def export_handle(self):
        buf = ctypes.create_string_buffer(64)
        _check(lib().w4a8_ipc_export(self.base, buf))
        return buf.raw

    def connect_handles(self, handles):
        """handles[r] = 64-byte CUDA IPC handle of rank r's arena (this rank's own entry is ignored)."""
        bases = (_P * self.world)()
        for r, hd in enumerate(handles):
            if r == self.rank:
                bases[r] = self.base
            else:
                p = _P()
                _check(lib().w4a8_ipc_open(hd, ctypes.byref(p)))
                self._opened.append(p)
                bases[r] = p.value
        _check(lib().w4a8_arena_connect(self.handle, bases))

    def connect_pointers(self, pointers):
        """pointers[r] = arena base of rank r already mapped into this process (same-process emulation, or another
        peer-mapping mechanism)."""
        bases = (_P * self.world)(*[int(p) for p in pointers])
        _check(lib().w4a8_arena_connect(self.handle, bases))

    def tensor(self, offset, shape, dtype=None):
        """A torch view of the local arena (no copy)."""
        import torch
        dtype = dtype or torch.float32
        return _as_tensor(self.base + offset, shape, dtype)

    def gemv_allgather(self, xq, xs, Wq, sw, y_offset, IN, rows, row0, ldY, S, scale_dtype, epoch, stream=None):
        _check(lib().w4a8_gemv_allgather(_ptr(xq), _ptr(xs), _ptr(Wq), _ptr(sw), self.handle, y_offset, IN, rows, row0, ldY, S,
                                         scale_dtype, epoch, _stream(stream)))

    def gemm_allgather(self, X, xs, Wq, sw, y_offset, M, rows, row0, ldY, K, scale_dtype, epoch, stream=None):
        _check(lib().w4a8_gemm_allgather(_ptr(X), _ptr(xs), _ptr(Wq), _ptr(sw), self.handle, y_offset, M, rows, row0, ldY, K,
                                         scale_dtype, epoch, _stream(stream)))

    def gemv_allgather_sync(self, xq, xs, Wq, sw, y_offset, IN, rows, row0, ldY, S, scale_dtype, epoch, timeout_us=1000000, stream=None):
        """gemv_allgather with the wait folded into its last kernel: when that kernel completes, Y is complete here."""
        _check(lib().w4a8_gemv_allgather_sync(_ptr(xq), _ptr(xs), _ptr(Wq), _ptr(sw), self.handle, y_offset, IN, rows, row0, ldY, S,
                                              scale_dtype, epoch, timeout_us, _stream(stream)))

    def gemm_allgather_sync(self, X, xs, Wq, sw, y_offset, M, rows, row0, ldY, K, scale_dtype, epoch, timeout_us=1000000, stream=None):
        _check(lib().w4a8_gemm_allgather_sync(_ptr(X), _ptr(xs), _ptr(Wq), _ptr(sw), self.handle, y_offset, M, rows, row0, ldY, K,
                                              scale_dtype, epoch, timeout_us, _stream(stream)))

    def wait(self, epoch, timeout_us=1000000, stream=None):
        _check(lib().w4a8_allgather_wait(self.handle, epoch, timeout_us, _stream(stream)))

    def advance_epoch(self, delta, stream=None):
        _check(lib().w4a8_arena_advance_epoch(self.handle, delta, _stream(stream)))

    def close(self):
        for p in self._opened:
            lib().w4a8_ipc_close(p)
        self._opened = []
        if self.handle:
            lib().w4a8_arena_destroy(self.handle)
            self.handle = None


def _as_tensor(ptr, shape, dtype):
    """Wraps raw device memory as a torch tensor through the CUDA array interface (no copy, no ownership)."""
    import torch
    typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1", torch.int8: "|i1"}[dtype]

    class _Holder:
        pass
    h = _Holder()
    h.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (int(ptr), False), "version": 3, "strides": None}
    return torch.as_tensor(h, device="cuda")
