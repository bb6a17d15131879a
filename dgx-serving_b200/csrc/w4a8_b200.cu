// The single translation unit of libw4a8_b200.so: includes every kernel file and defines the C ABI
// declared in include/w4a8_b200.h.  Build (see dgx-serving_b200/build.py):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -lineinfo -Xcompiler -fPIC -shared
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>

#include "common.cuh"
#include "quantize_x.cuh"
#include "fused_quantize.cuh"
#include "gemv_w4a8.cuh"
#include "gemv_w4a8_mma.cuh"
#include "gemv_w4a8_bulk.cuh"
#include "gemv_w4a8_tc.cuh"
#include "gemm_w4a8_tc.cuh"
#include "gemm_w4a8_tcf.cuh"
#include "moe_w4a8.cuh"

namespace w4a8 {

char *err_buf() {
    static thread_local char buf[512] = {0};
    return buf;
}

bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("W4A8_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}

int sm_count() {
    static int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

int require_sm100() {
    static int cached_dev = -1, cached_rc = W4A8_OK;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "no CUDA device (this library has no CPU path)");
    if (dev != cached_dev) {
        int major = 0;
        e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceGetAttribute");
        cached_rc = (major == 10) ? W4A8_OK : W4A8_ERR_UNSUPPORTED;
        cached_dev = dev;
        if (cached_rc != W4A8_OK)
            return fail(W4A8_ERR_UNSUPPORTED, "device %d is compute capability %d.x; this build targets sm_100a only", dev, major);
    }
    if (cached_rc != W4A8_OK) return fail(W4A8_ERR_UNSUPPORTED, "device %d is not an sm_100 device", dev);
    return W4A8_OK;
}

// Exact integer group dots through the dp4a path of the GEMV kernels: one thread per (m, n, group).
__global__ void __launch_bounds__(256) group_dots_dp4a_kernel(const int8_t *__restrict__ xq, const uint8_t *__restrict__ Wq,
                                                              int32_t *__restrict__ D, int M, int N, int K) {
    const int nb = K / QBLK;
    const long total = (long)M * N * nb;
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int b = (int)(i % nb);
        const long mn = i / nb;
        const int n = (int)(mn % N), m = (int)(mn / N);
        const uint32_t *w = reinterpret_cast<const uint32_t *>(Wq + (size_t)n * (K / 2) + 16 * b);
        const uint32_t *x = reinterpret_cast<const uint32_t *>(xq + (size_t)m * K + 32 * b);
        int d = 0;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t we, wo, xe, xo;
            unpack8_x16(w[c], we, wo);
            split_even_odd(x[2 * c], x[2 * c + 1], xe, xo);
            d = __dp4a((int)xe, (int)we, d);
            d = __dp4a((int)xo, (int)wo, d);
        }
        D[i] = d >> 4;
    }
}

static int check_common(const void *a, const void *b, const void *c, const void *d, const void *e, int K, int scale_dtype,
                        const char *who) {
    if (!a || !b || !c || !d || !e) return fail(W4A8_ERR_ARG, "%s: null pointer argument", who);
    if (K < 0 || K % QBLK != 0) return fail(W4A8_ERR_ARG, "%s: K=%d must be a non-negative multiple of %d", who, K, QBLK);
    if (scale_dtype != 0 && scale_dtype != 1) return fail(W4A8_ERR_ARG, "%s: scale_dtype=%d (0 fp32, 1 fp16)", who, scale_dtype);
    return W4A8_OK;
}

}  // namespace w4a8

using namespace w4a8;

#ifndef W4A8_GEMM_DEFAULT
#define W4A8_GEMM_DEFAULT 1
#endif

W4A8_API int w4a8_version(void) { return 100; }
W4A8_API const char *w4a8_last_error(void) { return err_buf(); }

W4A8_API int w4a8_device_status(uint32_t *detail) {
    unsigned int v = 0, zero = 0;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return cuda_fail(e, "cudaDeviceSynchronize");
    e = cudaMemcpyFromSymbol(&v, g_dev_error, sizeof(v));
    if (e != cudaSuccess) return cuda_fail(e, "read device error word");
    if (v != 0) {
        cudaMemcpyToSymbol(g_dev_error, &zero, sizeof(zero));
        if (detail) *detail = v;
        return fail(W4A8_ERR_DEVICE, "a kernel's bounded wait ran out (code 0x%x)", v);
    }
    if (detail) *detail = 0;
    return W4A8_OK;
}

W4A8_API int w4a8_quantize_x_q8(const float *X, int8_t *xq, float *xs, int32_t *xsum, int IN, int S, void *stream) {
    if (S < 0 || IN < 0 || IN % QBLK != 0) return fail(W4A8_ERR_ARG, "quantize_x_q8: IN=%d S=%d (IN must be a multiple of %d)", IN, S, QBLK);
    if (S == 0 || IN == 0) return W4A8_OK;
    if (!X || !xq || !xs) return fail(W4A8_ERR_ARG, "quantize_x_q8: null pointer argument");
    int rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    return launch_quantize_x(X, xq, xs, xsum, IN, S, (cudaStream_t)stream);
}

W4A8_API int w4a8_rmsnorm_quantize_x_q8(const float *X, const float *W, float eps, int variant, float *Y, int8_t *xq, float *xs,
                                        int32_t *xsum, int IN, int S, void *stream) {
    if (S < 0 || IN < 0 || IN % QBLK != 0) return fail(W4A8_ERR_ARG, "rmsnorm_quantize_x_q8: IN=%d S=%d (IN must be a multiple of %d)", IN, S, QBLK);
    if (variant < 0 || variant > 2) return fail(W4A8_ERR_ARG, "rmsnorm_quantize_x_q8: variant=%d (0 scale, 1 one-plus-scale, 2 no scale)", variant);
    if (S == 0 || IN == 0) return W4A8_OK;
    if (!X || !xq || !xs || (variant != 2 && !W)) return fail(W4A8_ERR_ARG, "rmsnorm_quantize_x_q8: null pointer argument");
    if (!aligned(X, 16) || !aligned(xq, 4) || (W && !aligned(W, 16)) || (Y && !aligned(Y, 16)))
        return fail(W4A8_ERR_ALIGN, "rmsnorm_quantize_x_q8: X, W and Y must be 16-byte aligned");
    int rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    return launch_rmsnorm_quantize(X, W, eps, variant, Y, xq, xs, xsum, IN, S, (cudaStream_t)stream);
}

W4A8_API int w4a8_glu_quantize_x_q8(const float *G, const float *U, int act, float *Y, int8_t *xq, float *xs, int32_t *xsum, int IN,
                                    int S, void *stream) {
    if (S < 0 || IN < 0 || IN % QBLK != 0) return fail(W4A8_ERR_ARG, "glu_quantize_x_q8: IN=%d S=%d (IN must be a multiple of %d)", IN, S, QBLK);
    if (act < 0 || act > 1) return fail(W4A8_ERR_ARG, "glu_quantize_x_q8: act=%d (0 SwiGLU, 1 GeGLU)", act);
    if (S == 0 || IN == 0) return W4A8_OK;
    if (!G || !U || !xq || !xs) return fail(W4A8_ERR_ARG, "glu_quantize_x_q8: null pointer argument");
    if (!aligned(G, 16) || !aligned(U, 16) || !aligned(xq, 4) || (Y && !aligned(Y, 16)))
        return fail(W4A8_ERR_ALIGN, "glu_quantize_x_q8: G, U and Y must be 16-byte aligned");
    int rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    return launch_glu_quantize(G, U, act, Y, xq, xs, xsum, IN, S, (cudaStream_t)stream);
}

// GEMV kernel policy: 0 auto, 1 always the dp4a kernel, 2 mma.sync tensor path for every S it supports, 3 bulk-copy
// stream for every single row it supports, 5 tcgen05 tensor path for every S it supports.  Initialised from the
// environment (W4A8_GEMV = dp4a | mma | bulk | tc), changed at run time with w4a8_config("gemv_kernel", v).
static int g_gemv_policy = -1;
static int gemv_policy() {
    if (g_gemv_policy < 0) {
        const char *e = getenv("W4A8_GEMV");
        g_gemv_policy = !e ? 0 : (e[0] == 'm' ? 2 : (e[0] == 'd' ? 1 : (e[0] == 'b' ? 3 : (e[0] == 't' ? 5 : 0))));
    }
    return g_gemv_policy;
}
static bool gemv_use_mma(int S, int scale_dtype) {
    const int p = gemv_policy();
    // auto: the dp4a streaming kernel only for a single row with fp32 scales, where it is the fastest; its two-byte
    // scale loads make it slower than the tensor-path kernel with fp16 scales
    return p == 2 || (p == 0 && (S >= 2 || scale_dtype == 1));
}

// The one place that decides which GEMV kernel runs and in how many launches.  count_only != nullptr: nothing is
// launched, *count_only receives the number of kernel launches the call would make.  `oa` carries the peer-store
// epilogue of the fused all-gather (oa.peers == nullptr: ordinary Y); the count and the launch are decided by this one
// function under the same arguments.
static int gemv_dispatch(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int IN, int OUT, int S,
                         int scale_dtype, cudaStream_t st, int *count_only, const OutArgs &oa_in = OutArgs()) {
    const int pol = gemv_policy();
    if (pol == 5 && gemv_tc::supported(xq, Wq, sw, IN, S < 16 ? S : 16, scale_dtype)) {
        // tcgen05 path (opt-in): rows in passes of up to 16, MMQ order for every S
        if (count_only) { *count_only = (S + 15) / 16; return W4A8_OK; }
        for (int s0 = 0; s0 < S; s0 += 16) {
            const int s = S - s0 < 16 ? S - s0 : 16;
            OutArgs oa = oa_in;
            if (oa.peers) oa.y_off += (size_t)s0 * oa.ld * sizeof(float);
            int rc = gemv_tc::launch(xq + (size_t)s0 * IN, xs + (size_t)s0 * (IN / QBLK), Wq, sw, Y + (size_t)s0 * OUT, IN, OUT, s,
                                     scale_dtype, st, oa);
            if (rc != W4A8_OK) return rc;
        }
        return W4A8_OK;
    }
    // One row.  The bulk-copy stream and the dp4a kernel give the same bits; which is faster depends on the matrix: the
    // bulk-copy stream has the higher steady rate (6.5-6.9 TB/s against 6.0) and the larger fixed cost per launch
    // (about 2.7 against 1.1 us), so auto takes it from 96 MB of weights up (K=5120: N >= 30k, an lm_head) and for
    // fp16 scales, whose two-byte loads slow the dp4a kernel down; a 56 MB MLP matrix stays on the dp4a kernel
    // (10.7 against 11.0 us).  Rows shorter than 2048 elements make the bulk copies too small.  With the peer-store
    // epilogue (a rank's slice of an N-sharded matrix) the dp4a kernel's smaller fixed cost wins as well.
    const size_t wbytes = (size_t)OUT * ((size_t)IN / 2 + (size_t)(IN / QBLK) * (scale_dtype == 1 ? 2 : 4));
    const bool bulk_auto = IN >= 2048 && !oa_in.peers && (scale_dtype == 1 || wbytes >= ((size_t)96 << 20));
    if (S == 1 && (pol == 3 || (pol == 0 && bulk_auto))) {
        gemv_bulk::Plan bp;
        if (gemv_bulk::plan_for(xq, Wq, sw, IN, scale_dtype, &bp)) {
            if (count_only) { *count_only = 1; return W4A8_OK; }
            return gemv_bulk::launch(xq, xs, Wq, sw, Y, IN, OUT, scale_dtype, bp, st, oa_in);
        }
    }
    if (gemv_use_mma(S, scale_dtype)) {
        // rows go in passes of up to 16 (8 when 16 rows of activations do not fit in shared memory next to the ring)
        gemv_mma::Plan plan;
        int per = S < 16 ? S : 16;
        bool ok = gemv_mma::plan_for(Wq, sw, IN, per, &plan);
        if (!ok && per > 8) { per = 8; ok = gemv_mma::plan_for(Wq, sw, IN, per, &plan); }
        if (ok) {
            if (count_only) { *count_only = (S + per - 1) / per; return W4A8_OK; }
            for (int s0 = 0; s0 < S; s0 += per) {
                const int s = S - s0 < per ? S - s0 : per;
                gemv_mma::Plan pl = plan;
                if (s <= 8 && pl.MH == 2) gemv_mma::plan_for(Wq, sw, IN, s, &pl);
                OutArgs oa = oa_in;
                if (oa.peers) oa.y_off += (size_t)s0 * oa.ld * sizeof(float);
                int rc = gemv_mma::launch(xq + (size_t)s0 * IN, xs + (size_t)s0 * (IN / QBLK), Wq, sw, Y + (size_t)s0 * OUT, IN, OUT, s,
                                          scale_dtype, pl, st, oa);
                if (rc != W4A8_OK) return rc;
            }
            return W4A8_OK;
        }
    }
    if (count_only) { *count_only = (S + GEMV_MT_MAX - 1) / GEMV_MT_MAX; return W4A8_OK; }
    return launch_gemv(xq, xs, Wq, sw, Y, IN, OUT, S, scale_dtype, st, oa_in);
}

// GEMM kernel policy: 0 = fp16-operand tensor-core kernel (kind::f16, exact float group dots), 1 = int8-operand kernel
// (kind::i8, int32 group dots).  Same results bit for bit.  Environment W4A8_GEMM = f16 | i8.
static int g_gemm_policy = -1;
static int gemm_policy() {
    if (g_gemm_policy < 0) {
        const char *e = getenv("W4A8_GEMM");
        g_gemm_policy = !e ? W4A8_GEMM_DEFAULT : (e[0] == 'i' ? 1 : 0);
    }
    return g_gemm_policy;
}
static int gemm_launch(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int M, int N, int K,
                       int scale_dtype, int nsplit, int gsplit, cudaStream_t st) {
    if (gemm_policy() == 1) return gemm::launch_tc(X, xs, Wq, sw, Y, M, N, K, scale_dtype, nsplit, gsplit, st, OutArgs());
    return gemmf::launch(X, xs, Wq, sw, Y, M, N, K, scale_dtype, nsplit, gsplit, st);
}

static int g_moe_policy = 0;   // w4a8_moe_block: 0 auto (by slot count), 1 grouped GEMV, 2 sorted grouped GEMM

W4A8_API int w4a8_config(const char *key, int value) {
    if (!key) return fail(W4A8_ERR_ARG, "config: null key");
    if (!strcmp(key, "gemm_kernel")) {
        if (value < 0 || value > 1) return fail(W4A8_ERR_ARG, "config: gemm_kernel = 0 (fp16 operands), 1 (int8 operands); got %d", value);
        g_gemm_policy = value;
        return W4A8_OK;
    }
    if (!strcmp(key, "gemv_kernel")) {
        if (value < 0 || value > 5 || value == 4)
            return fail(W4A8_ERR_ARG, "config: gemv_kernel = 0 (auto), 1 (dp4a), 2 (mma.sync tensor path), 3 (bulk-copy stream for S = 1), 5 (tcgen05 tensor path); got %d", value);
        g_gemv_policy = value;
        return W4A8_OK;
    }
    if (!strcmp(key, "moe_kernel")) {
        if (value < 0 || value > 2) return fail(W4A8_ERR_ARG, "config: moe_kernel = 0 (auto), 1 (grouped GEMV), 2 (sorted grouped GEMM); got %d", value);
        g_moe_policy = value;
        return W4A8_OK;
    }
    return fail(W4A8_ERR_ARG, "config: unknown key '%s'", key);
}

W4A8_API int w4a8_gemv(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int IN, int OUT,
                       int S, int scale_dtype, void *stream) {
    if (S < 0 || OUT < 0) return fail(W4A8_ERR_ARG, "gemv: negative size S=%d OUT=%d", S, OUT);
    if (S == 0 || OUT == 0) return W4A8_OK;
    int rc = check_common(xq, xs, Wq, sw, Y, IN, scale_dtype, "gemv");
    if (rc != W4A8_OK) return rc;
    if (!aligned(xq, 4) || !aligned(Wq, 4)) return fail(W4A8_ERR_ALIGN, "gemv: xq and Wq must be 4-byte aligned");
    rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    if (IN == 0) {
        cudaError_t e = cudaMemsetAsync(Y, 0, (size_t)S * OUT * sizeof(float), (cudaStream_t)stream);
        return e == cudaSuccess ? W4A8_OK : cuda_fail(e, "gemv: memset");
    }
    return gemv_dispatch(xq, xs, Wq, sw, Y, IN, OUT, S, scale_dtype, (cudaStream_t)stream, nullptr);
}

W4A8_API int w4a8_gemv_multi(const int8_t *xq, const float *xs, int count, const uint8_t *const *Wq, const void *const *sw,
                             float *const *Y, const int *OUT, int IN, int S, int scale_dtype, void *stream) {
    if (count < 0 || count > gemv_bulk::MAX_MATS) return fail(W4A8_ERR_ARG, "gemv_multi: count=%d (0..%d)", count, gemv_bulk::MAX_MATS);
    if (count == 0 || S == 0) return W4A8_OK;
    if (!Wq || !sw || !Y || !OUT) return fail(W4A8_ERR_ARG, "gemv_multi: null array argument");
    // One launch when every matrix can take the bulk-copy stream (one row, the auto policy's conditions); else the
    // matrices go one after the other through w4a8_gemv.  Either way each output equals w4a8_gemv's, bit for bit.
    bool one = S == 1 && (gemv_policy() == 3 || (gemv_policy() == 0 && IN >= 2048));
    gemv_bulk::Plan bp;
    gemv_bulk::Mats m = {};
    for (int i = 0; i < count && one; i++) {
        if (OUT[i] <= 0 || !Wq[i] || !sw[i] || !Y[i] || !xq || !xs) { one = false; break; }
        gemv_bulk::Plan pi;
        if (!gemv_bulk::plan_for(xq, Wq[i], sw[i], IN, scale_dtype, &pi)) { one = false; break; }
        bp = pi;
        m.Wq[i] = Wq[i]; m.sw[i] = sw[i]; m.Y[i] = Y[i]; m.OUT[i] = OUT[i];
    }
    if (one) {
        if (scale_dtype != 0 && scale_dtype != 1) return fail(W4A8_ERR_ARG, "gemv_multi: scale_dtype=%d", scale_dtype);
        int rc = require_sm100();
        if (rc != W4A8_OK) return rc;
        m.count = count;
        return gemv_bulk::launch_multi(xq, xs, m, IN, scale_dtype, bp, (cudaStream_t)stream);
    }
    for (int i = 0; i < count; i++) {
        int rc = w4a8_gemv(xq, xs, Wq[i], sw[i], Y[i], IN, OUT[i], S, scale_dtype, stream);
        if (rc != W4A8_OK) return rc;
    }
    return W4A8_OK;
}

W4A8_API int w4a8_gemm(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int M, int N, int K,
                       int scale_dtype, void *stream) {
    if (M < 0 || N < 0) return fail(W4A8_ERR_ARG, "gemm: negative size M=%d N=%d", M, N);
    if (M == 0 || N == 0) return W4A8_OK;   // reference: kernels/gemm_mmq_raster.cuh:118
    int rc = check_common(X, xs, Wq, sw, Y, K, scale_dtype, "gemm");
    if (rc != W4A8_OK) return rc;
    if (!aligned(X, 16) || !aligned(Wq, 16))
        return fail(W4A8_ERR_ALIGN, "gemm: X and Wq must be 16-byte aligned (TMA); use w4a8_gemv for unaligned operands");
    rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    if (K == 0) {
        cudaError_t e = cudaMemsetAsync(Y, 0, (size_t)M * N * sizeof(float), (cudaStream_t)stream);
        return e == cudaSuccess ? W4A8_OK : cuda_fail(e, "gemm: memset");
    }
    return gemm_launch(X, xs, Wq, sw, Y, M, N, K, scale_dtype, 1, K / QBLK, (cudaStream_t)stream);
}

// Split count and groups per split.  Boundaries follow the reference: K-tiles of 64 (2 groups), ranges of
// ceil(niter/splitk) K-tiles (kernels/gemm_mmq.cuh:138-139), default split count ~96 CTAs clamp 1..8 (:209-210).
constexpr int SPLITK_MAX = 4096;   // explicit split counts above this are refused (K = 131072 has 2048 K-tiles of 64)
static void splitk_plan(int N, int K, int splitk_in, int *nsplit, int *gsplit) {
    const int nb = K / QBLK;
    const int niter = (nb + 1) / 2;
    int sk = splitk_in;
    if (sk <= 0) {
        const int ntile = (N + 127) / 128;
        const int want = 96 / ntile;
        sk = want > 1 ? (want < 8 ? want : 8) : 1;
    }
    const int itper = (niter + sk - 1) / sk;
    *nsplit = sk;
    *gsplit = (itper > 0 ? itper : 1) * 2;
}

W4A8_API size_t w4a8_gemm_splitk_workspace_bytes(int M, int N, int K, int splitk) {
    if (M <= 0 || N <= 0 || K <= 0 || splitk > SPLITK_MAX) return 0;
    int ns, gs;
    splitk_plan(N, K, splitk, &ns, &gs);
    return ns > 1 ? (size_t)ns * M * N * sizeof(float) : 0;
}

W4A8_API int w4a8_gemm_splitk(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int M, int N,
                              int K, int scale_dtype, int splitk, void *workspace, size_t workspace_bytes, void *stream) {
    if (M < 0 || N < 0) return fail(W4A8_ERR_ARG, "gemm_splitk: negative size M=%d N=%d", M, N);
    if (splitk > SPLITK_MAX) return fail(W4A8_ERR_ARG, "gemm_splitk: splitk=%d (0 = automatic, at most %d)", splitk, SPLITK_MAX);
    if (M == 0 || N == 0) return W4A8_OK;
    int rc = check_common(X, xs, Wq, sw, Y, K, scale_dtype, "gemm_splitk");
    if (rc != W4A8_OK) return rc;
    if (!aligned(X, 16) || !aligned(Wq, 16)) return fail(W4A8_ERR_ALIGN, "gemm_splitk: X and Wq must be 16-byte aligned (TMA)");
    if (K == 0) return w4a8_gemm(X, xs, Wq, sw, Y, M, N, K, scale_dtype, stream);
    rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    int ns, gs;
    splitk_plan(N, K, splitk, &ns, &gs);
    cudaStream_t st = (cudaStream_t)stream;
    if (ns == 1) return gemm_launch(X, xs, Wq, sw, Y, M, N, K, scale_dtype, 1, K / QBLK, st);
    const size_t need = (size_t)ns * M * N * sizeof(float);
    if (!workspace || workspace_bytes < need)
        return fail(W4A8_ERR_WORKSPACE, "gemm_splitk: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    if (!aligned(workspace, 16)) return fail(W4A8_ERR_ALIGN, "gemm_splitk: workspace must be 16-byte aligned");
    rc = gemm_launch(X, xs, Wq, sw, (float *)workspace, M, N, K, scale_dtype, ns, gs, st);
    if (rc != W4A8_OK) return rc;
    const long MN = (long)M * N;
    long want = (MN + 255) / 256, cap = (long)sm_count() * 8;
    gemm::splitk_reduce_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>((const float *)workspace, Y, MN, ns);
    return launch_status("splitk_reduce");
}

// ---- split-K without an allocator ---------------------------------------------------------------------
// Partial-sum buffer for w4a8_gemm_splitk_static: lives in the library image, so no call ever allocates.
// In host code this name is only a handle for cudaGetSymbolAddress, never a usable pointer.
static __device__ __align__(256) float g_splitk_static_scratch[W4A8_SPLITK_STATIC_BYTES / sizeof(float)];

// Device address of the buffer on the current device; queried once per device and cached.  The query itself is not a
// stream operation, but the first call on a device also loads the module and configures the kernels, which a stream
// capture in progress does not allow: that case is refused with a message instead of failing somewhere inside.
static int splitk_static_ptr(float **out, cudaStream_t st) {
    constexpr int MAX_DEV = 64;
    static float *cached[MAX_DEV] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "gemm_splitk_static: cudaGetDevice");
    if (dev < 0 || dev >= MAX_DEV) return fail(W4A8_ERR_UNSUPPORTED, "gemm_splitk_static: device index %d out of range", dev);
    if (!cached[dev]) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        e = cudaStreamIsCapturing(st, &cs);
        if (e != cudaSuccess) return cuda_fail(e, "gemm_splitk_static: cudaStreamIsCapturing");
        if (cs != cudaStreamCaptureStatusNone)
            return fail(W4A8_ERR_UNSUPPORTED, "gemm_splitk_static: the first call on a device must not be made while the stream is "
                                              "being captured (it looks up the built-in buffer); call it once outside the capture first");
        float *p = nullptr;
        e = cudaGetSymbolAddress((void **)&p, g_splitk_static_scratch);
        if (e != cudaSuccess || !p) return cuda_fail(e, "gemm_splitk_static: cudaGetSymbolAddress");
        cached[dev] = p;
    }
    *out = cached[dev];
    return W4A8_OK;
}

W4A8_API int w4a8_gemm_splitk_static(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int M, int N,
                                     int K, int scale_dtype, int splitk, void *stream) {
    if (M < 0 || N < 0) return fail(W4A8_ERR_ARG, "gemm_splitk_static: negative size M=%d N=%d", M, N);
    if (splitk > SPLITK_MAX) return fail(W4A8_ERR_ARG, "gemm_splitk_static: splitk=%d (0 = automatic, at most %d)", splitk, SPLITK_MAX);
    if (M == 0 || N == 0) return W4A8_OK;
    int rc = check_common(X, xs, Wq, sw, Y, K, scale_dtype, "gemm_splitk_static");
    if (rc != W4A8_OK) return rc;
    if (!aligned(X, 16) || !aligned(Wq, 16)) return fail(W4A8_ERR_ALIGN, "gemm_splitk_static: X and Wq must be 16-byte aligned (TMA)");
    if (K == 0) return w4a8_gemm(X, xs, Wq, sw, Y, M, N, K, scale_dtype, stream);
    int ns, gs;
    splitk_plan(N, K, splitk, &ns, &gs);
    const size_t need = (size_t)ns * M * N * sizeof(float);
    if (ns > 1 && need > (size_t)W4A8_SPLITK_STATIC_BYTES)
        return fail(W4A8_ERR_UNSUPPORTED,
                    "gemm_splitk_static: %d splits x M=%d x N=%d need %zu bytes of partial sums, the built-in buffer holds %u; "
                    "use w4a8_gemm_splitk with a caller-owned workspace",
                    ns, M, N, need, (unsigned)W4A8_SPLITK_STATIC_BYTES);
    rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (ns == 1) return gemm_launch(X, xs, Wq, sw, Y, M, N, K, scale_dtype, 1, K / QBLK, st);
    float *scratch = nullptr;
    rc = splitk_static_ptr(&scratch, st);
    if (rc != W4A8_OK) return rc;
    // kernel 1 writes every partial sum [split][m][n], m < M, n < N (an empty K range writes zeros), kernel 2 reads
    // exactly those: nothing left over from an earlier call is ever read, so nothing needs clearing.
    rc = gemm_launch(X, xs, Wq, sw, scratch, M, N, K, scale_dtype, ns, gs, st);
    if (rc != W4A8_OK) return rc;
    const long MN = (long)M * N;
    long want = (MN + 255) / 256, cap = (long)sm_count() * 8;
    gemm::splitk_reduce_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(scratch, Y, MN, ns);
    return launch_status("splitk_reduce (static)");
}

W4A8_API int w4a8_group_dots(const int8_t *xq, const uint8_t *Wq, int32_t *D, int M, int N, int K, int path, void *stream) {
    if (M < 0 || N < 0 || K < 0 || K % QBLK != 0) return fail(W4A8_ERR_ARG, "group_dots: bad shape M=%d N=%d K=%d", M, N, K);
    if (M == 0 || N == 0 || K == 0) return W4A8_OK;
    if (!xq || !Wq || !D) return fail(W4A8_ERR_ARG, "group_dots: null pointer argument");
    int rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (path == 1) {
        if (!aligned(xq, 16) || !aligned(Wq, 16)) return fail(W4A8_ERR_ALIGN, "group_dots: tensor-core path needs 16-byte aligned operands");
        return gemm::launch_tc_dump(xq, Wq, D, M, N, K, st);
    }
    if (path == 2) {
        if (!aligned(xq, 16) || !aligned(Wq, 16)) return fail(W4A8_ERR_ALIGN, "group_dots: tensor-core path needs 16-byte aligned operands");
        return gemmf::launch_dump(xq, Wq, D, M, N, K, st);
    }
    if (path != 0) return fail(W4A8_ERR_ARG, "group_dots: path=%d (0 dp4a, 1 tcgen05 int8, 2 tcgen05 fp16)", path);
    if (!aligned(xq, 4) || !aligned(Wq, 4)) return fail(W4A8_ERR_ALIGN, "group_dots: operands must be 4-byte aligned");
    const long total = (long)M * N * (K / QBLK);
    long want = (total + 255) / 256, cap = (long)sm_count() * 8;
    group_dots_dp4a_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(xq, Wq, D, M, N, K);
    return launch_status("group_dots");
}

W4A8_API int w4a8_linear(const float *X, int8_t *xq, float *xs, int32_t *xsum, const uint8_t *Wq, const void *sw, float *Y,
                         int S, int N, int K, int scale_dtype, int skip_quantize, void *stream) {
    if (!skip_quantize) {
        int rc = w4a8_quantize_x_q8(X, xq, xs, xsum, K, S, stream);
        if (rc != W4A8_OK) return rc;
    }
    if (S <= 16 || !aligned(xq, 16) || !aligned(Wq, 16)) return w4a8_gemv(xq, xs, Wq, sw, Y, K, N, S, scale_dtype, stream);
    return w4a8_gemm(xq, xs, Wq, sw, Y, S, N, K, scale_dtype, stream);
}

// Device alias of a host pointer that the GPU can address directly (pinned and mapped; with unified addressing every
// cudaHostAlloc / cudaHostRegister range is), else nullptr.
static void *mapped_alias(const void *host) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, host) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return (a.type == cudaMemoryTypeHost) ? a.devicePointer : nullptr;
}
W4A8_API int w4a8_linear_host(const float *X_host, float *Y_host, float *X_dev, int8_t *xq, float *xs, int32_t *xsum, float *Y_dev,
                              const uint8_t *Wq, const void *sw, int S, int N, int K, int scale_dtype, void *stream) {
    if (S < 0 || N < 0 || K < 0) return fail(W4A8_ERR_ARG, "linear_host: negative size");
    if (S == 0 || N == 0) return W4A8_OK;
    if (!X_host || !Y_host || !X_dev || !Y_dev) return fail(W4A8_ERR_ARG, "linear_host: null buffer");
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    // A small step (decode) whose X is pinned, mapped host memory skips the host-to-device copy: quantize_x reads X over
    // the bus itself, which saves a stream operation worth more than the 20 KB transfer (48 -> 35 us per step on the
    // headline shape).  The results still leave through the copy engine: a kernel writing them to host memory
    // (coalesced, or straight from the GEMV epilogue) measured no faster.
    const size_t xbytes = (size_t)S * K * sizeof(float), ybytes = (size_t)S * N * sizeof(float);
    const float *X_in = X_dev;
    if (xbytes <= (1u << 20))
        if (void *xa = mapped_alias(X_host)) X_in = static_cast<const float *>(xa);
    if (X_in == X_dev) {
        e = cudaMemcpyAsync(X_dev, X_host, xbytes, cudaMemcpyHostToDevice, st);
        if (e != cudaSuccess) return cuda_fail(e, "linear_host: H2D");
    }
    int rc = w4a8_linear(X_in, xq, xs, xsum, Wq, sw, Y_dev, S, N, K, scale_dtype, 0, stream);
    if (rc != W4A8_OK) return rc;
    e = cudaMemcpyAsync(Y_host, Y_dev, ybytes, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? W4A8_OK : cuda_fail(e, "linear_host: D2H");
}

W4A8_API int w4a8_moe_gemv(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, const int32_t *idx, float *Y,
                           int nslots, int topk, int x_per_slot, int N, int K, int num_experts, int scale_dtype, void *stream) {
    if (nslots < 0 || N < 0 || topk <= 0 || num_experts <= 0)
        return fail(W4A8_ERR_ARG, "moe_gemv: bad sizes nslots=%d N=%d topk=%d experts=%d", nslots, N, topk, num_experts);
    if (nslots == 0 || N == 0) return W4A8_OK;
    int rc = check_common(xq, xs, Wq, sw, Y, K, scale_dtype, "moe_gemv");
    if (rc != W4A8_OK) return rc;
    if (!idx) return fail(W4A8_ERR_ARG, "moe_gemv: null expert index");
    if (K == 0) return fail(W4A8_ERR_ARG, "moe_gemv: K must be positive");
    if (!aligned(xq, 4) || !aligned(Wq, 4)) return fail(W4A8_ERR_ALIGN, "moe_gemv: xq and Wq must be 4-byte aligned");
    rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    return launch_moe_gemv(xq, xs, Wq, sw, idx, Y, nslots, topk, x_per_slot, N, K, num_experts, scale_dtype, (cudaStream_t)stream);
}

// ---- N-sharded weight upload ---------------------------------------------------------------------------
W4A8_API int w4a8_shard_rows(int64_t N, int rank, int world, int64_t *row0, int64_t *rows) {
    if (N < 0 || world <= 0 || rank < 0 || rank >= world || !row0 || !rows)
        return fail(W4A8_ERR_ARG, "shard_rows: N=%lld rank=%d world=%d", (long long)N, rank, world);
    const int64_t base = N / world, rem = N % world;
    const int64_t first_big = world - rem;   // ranks >= first_big hold base+1 rows
    *rows = base + (rank >= first_big ? 1 : 0);
    *row0 = base * rank + (rank > first_big ? rank - first_big : 0);
    return W4A8_OK;
}

static int upload_range(void **dev, const void *host, size_t bytes, const char *what) {
    *dev = nullptr;
    if (bytes == 0) return W4A8_OK;
    cudaError_t e = cudaMalloc(dev, bytes);
    if (e != cudaSuccess) return cuda_fail(e, what);
    e = cudaMemcpy(*dev, host, bytes, cudaMemcpyHostToDevice);
    // A copy from pageable memory may return before the DMA has landed.  The product kernels prefetch weights
    // ahead of their stream dependency (programmatic dependent launch), so the upload ends with the data in place.
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { cudaFree(*dev); *dev = nullptr; return cuda_fail(e, what); }
    return W4A8_OK;
}

static int shard_shape(int64_t N, int64_t K, int scale_dtype, int rank, int world, w4a8_qmat *out, const char *who) {
    if (!out) return fail(W4A8_ERR_ARG, "%s: null output", who);
    memset(out, 0, sizeof(*out));
    if (N < 0 || K < 0 || K % QBLK != 0) return fail(W4A8_ERR_ARG, "%s: bad shape N=%lld K=%lld", who, (long long)N, (long long)K);
    if (scale_dtype != 0 && scale_dtype != 1) return fail(W4A8_ERR_ARG, "%s: scale_dtype=%d", who, scale_dtype);
    int rc = w4a8_shard_rows(N, rank, world, &out->row0, &out->rows);
    if (rc != W4A8_OK) return rc;
    out->N = N; out->K = K; out->scale_dtype = scale_dtype;
    return W4A8_OK;
}

W4A8_API int w4a8_upload_qmat_shard(const uint8_t *host_wq, const void *host_sc, int64_t N, int64_t K, int scale_dtype, int rank,
                                    int world, w4a8_qmat *out) {
    int rc = shard_shape(N, K, scale_dtype, rank, world, out, "upload_qmat_shard");
    if (rc != W4A8_OK) return rc;
    if (!host_wq || !host_sc) return fail(W4A8_ERR_ARG, "upload_qmat_shard: null host pointer");
    const size_t esz = scale_dtype == 1 ? 2 : 4;
    const size_t wrow = (size_t)K / 2, srow = (size_t)(K / QBLK) * esz;
    rc = upload_range((void **)&out->wq, host_wq + (size_t)out->row0 * wrow, (size_t)out->rows * wrow, "upload q4 rows");
    if (rc != W4A8_OK) return rc;
    rc = upload_range(&out->sc, (const uint8_t *)host_sc + (size_t)out->row0 * srow, (size_t)out->rows * srow, "upload scale rows");
    if (rc != W4A8_OK) { cudaFree(out->wq); out->wq = nullptr; }
    return rc;
}

// Reads bytes [off, off+bytes) of `path` into a host buffer and uploads them.
static int load_range(const char *path, size_t off, size_t bytes, size_t file_need, void **dev) {
    *dev = nullptr;
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(W4A8_ERR_IO, "cannot open %s: %s", path, strerror(errno));
    struct stat sb;
    if (fstat(fd, &sb) != 0 || (size_t)sb.st_size < file_need) {
        close(fd);
        return fail(W4A8_ERR_IO, "%s: size mismatch (%lld bytes, need %zu)", path, (long long)sb.st_size, file_need);
    }
    if (bytes == 0) { close(fd); return W4A8_OK; }
    void *host = nullptr;
    cudaError_t e = cudaMallocHost(&host, bytes);
    if (e != cudaSuccess) { close(fd); return cuda_fail(e, "pinned staging buffer"); }
    size_t done = 0;
    while (done < bytes) {
        ssize_t r = pread(fd, (char *)host + done, bytes - done, (off_t)(off + done));
        if (r <= 0) { close(fd); cudaFreeHost(host); return fail(W4A8_ERR_IO, "%s: short read at %zu", path, off + done); }
        done += (size_t)r;
    }
    posix_fadvise(fd, (off_t)off, (off_t)bytes, POSIX_FADV_DONTNEED);   // like runtime/weights_qwen.cu:18
    close(fd);
    int rc = upload_range(dev, host, bytes, path);
    cudaFreeHost(host);
    return rc;
}

W4A8_API int w4a8_load_qmat_shard(const char *q4_path, const char *scale_path, int64_t N, int64_t K, int scale_dtype, int rank,
                                  int world, w4a8_qmat *out) {
    int rc = shard_shape(N, K, scale_dtype, rank, world, out, "load_qmat_shard");
    if (rc != W4A8_OK) return rc;
    if (!q4_path || !scale_path) return fail(W4A8_ERR_ARG, "load_qmat_shard: null path");
    const size_t esz = scale_dtype == 1 ? 2 : 4;
    const size_t wrow = (size_t)K / 2, srow = (size_t)(K / QBLK) * esz;
    rc = load_range(q4_path, (size_t)out->row0 * wrow, (size_t)out->rows * wrow, (size_t)N * wrow, (void **)&out->wq);
    if (rc != W4A8_OK) return rc;
    rc = load_range(scale_path, (size_t)out->row0 * srow, (size_t)out->rows * srow, (size_t)N * srow, &out->sc);
    if (rc != W4A8_OK) { cudaFree(out->wq); out->wq = nullptr; }
    return rc;
}

W4A8_API int w4a8_free_qmat(w4a8_qmat *m) {
    if (!m) return W4A8_OK;
    if (m->wq) cudaFree(m->wq);
    if (m->sc) cudaFree(m->sc);
    m->wq = nullptr;
    m->sc = nullptr;
    return W4A8_OK;
}

// ---- arenas, IPC, fused GEMV + all-gather ---------------------------------------------------------------------
struct w4a8_arena {
    unsigned char *base = nullptr;      // local allocation: user bytes + PEER_TAIL + two slot buffers
    size_t bytes = 0;                   // user bytes
    int rank = 0, world = 1;
    PeerDesc *desc_dev = nullptr;       // device copy of the descriptor (valid after connect)
    bool connected = false;
};

W4A8_API int w4a8_arena_create(size_t bytes, int rank, int world, w4a8_arena **out) {
    if (!out || world < 1 || world > PEER_MAX || rank < 0 || rank >= world)
        return fail(W4A8_ERR_ARG, "arena_create: rank=%d world=%d (1..%d ranks)", rank, world, PEER_MAX);
    int rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    w4a8_arena *a = new w4a8_arena();
    a->bytes = (bytes + 255) & ~(size_t)255;
    a->rank = rank; a->world = world;
    const size_t total = a->bytes + PEER_TAIL + 2 * LL_BUF_BYTES;
    cudaError_t e = cudaMalloc((void **)&a->base, total);
    if (e == cudaSuccess) e = cudaMemset(a->base, 0, total);
    if (e == cudaSuccess) e = cudaMalloc((void **)&a->desc_dev, sizeof(PeerDesc));
    if (e != cudaSuccess) { if (a->base) cudaFree(a->base); delete a; return cuda_fail(e, "arena_create"); }
    *out = a;
    return W4A8_OK;
}
W4A8_API void *w4a8_arena_base(w4a8_arena *a) { return a ? a->base : nullptr; }

W4A8_API int w4a8_arena_connect(w4a8_arena *a, void *const *bases) {
    if (!a || !bases) return fail(W4A8_ERR_ARG, "arena_connect: null argument");
    PeerDesc d = {};
    for (int r = 0; r < a->world; r++) {
        d.base[r] = (r == a->rank) ? a->base : (unsigned char *)bases[r];
        if (!d.base[r]) return fail(W4A8_ERR_ARG, "arena_connect: no mapping for rank %d", r);
    }
    d.flag_off = a->bytes;
    d.ll_off = a->bytes + PEER_TAIL;
    d.counter = reinterpret_cast<unsigned int *>(a->base + a->bytes + PEER_MAX * sizeof(unsigned int));
    d.epoch_base = d.counter + 1;
    d.world = a->world; d.rank = a->rank;
    cudaError_t e = cudaMemcpy(a->desc_dev, &d, sizeof(d), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return cuda_fail(e, "arena_connect");
    a->connected = true;
    return W4A8_OK;
}

W4A8_API int w4a8_arena_destroy(w4a8_arena *a) {
    if (!a) return W4A8_OK;
    if (a->desc_dev) cudaFree(a->desc_dev);
    if (a->base) cudaFree(a->base);
    delete a;
    return W4A8_OK;
}

W4A8_API int w4a8_ipc_export(void *dev_ptr, unsigned char handle[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handle size");
    if (!dev_ptr || !handle) return fail(W4A8_ERR_ARG, "ipc_export: null argument");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, dev_ptr);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcGetMemHandle");
    memcpy(handle, &h, 64);
    return W4A8_OK;
}
W4A8_API int w4a8_ipc_open(const unsigned char handle[64], void **dev_ptr) {
    if (!dev_ptr || !handle) return fail(W4A8_ERR_ARG, "ipc_open: null argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    cudaError_t e = cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return cuda_fail(e, "cudaIpcOpenMemHandle");
    return W4A8_OK;
}
W4A8_API int w4a8_ipc_close(void *dev_ptr) {
    if (!dev_ptr) return W4A8_OK;
    cudaError_t e = cudaIpcCloseMemHandle(dev_ptr);
    return e == cudaSuccess ? W4A8_OK : cuda_fail(e, "cudaIpcCloseMemHandle");
}

// Sends the finished slice on with the many-CTA copy kernel and publishes (and, wait_limit > 0, waits).
static int launch_scatter(w4a8_arena *a, size_t y_offset, int M, int ldY, int row0, int rows, uint32_t epoch, long long wait_limit,
                          cudaStream_t st) {
    const long units = (long)M * ((((long)ldY | row0 | rows) & 3) == 0 ? rows / 4 : rows);
    long want = (units + 255) / 256, cap = (long)sm_count() * 4;
    const unsigned grid = (unsigned)(want < cap ? (want > 0 ? want : 1) : cap);
    cudaError_t le = launch_pdl(allgather_scatter_kernel, dim3(grid), dim3(256), 0, st, (const PeerDesc *)a->desc_dev, y_offset, M, (long)ldY,
                                (long)row0, rows, (unsigned int)epoch, wait_limit);
    if (le != cudaSuccess) return cuda_fail(le, "allgather_scatter launch");
    return launch_status("allgather_scatter");
}
static long long wait_cycles(int timeout_us) {
    if (timeout_us <= 0) timeout_us = 1000000;
    return (long long)timeout_us * 2000;                 // SM clock <= 2 GHz: at least timeout_us
}

static int gemv_allgather_impl(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a, size_t y_offset,
                               int IN, int rows, int row0, int ldY, int S, int scale_dtype, uint32_t epoch, long long wait_limit,
                               cudaStream_t st) {
    if (!a || !a->connected) return fail(W4A8_ERR_ARG, "gemv_allgather: arena not connected");
    if (S < 0 || rows < 0 || row0 < 0 || ldY < row0 + rows) return fail(W4A8_ERR_ARG, "gemv_allgather: bad shape S=%d rows=%d row0=%d ldY=%d", S, rows, row0, ldY);
    if (y_offset % 16 != 0 || y_offset + (size_t)S * ldY * sizeof(float) > a->bytes)
        return fail(W4A8_ERR_ARG, "gemv_allgather: Y[%d x %d] at offset %zu does not fit the %zu-byte arena", S, ldY, y_offset, a->bytes);
    if (IN <= 0) return fail(W4A8_ERR_ARG, "gemv_allgather: IN must be positive");
    float *Ylocal = reinterpret_cast<float *>(a->base + y_offset);   // unused by the peer path; keeps the argument checks happy
    static const int mode = [] { const char *e = getenv("W4A8_ALLGATHER"); return !e ? 0 : e[0] == 'p' ? 1 : e[0] == 'f' ? 2 : e[0] == 's' ? 3 : 0; }();
    OutArgs oa;
    oa.peers = a->desc_dev; oa.y_off = y_offset; oa.ld = ldY; oa.col0 = row0; oa.epoch = epoch;
    oa.local_only = 1; oa.M = S; oa.cols = rows;
    // how many launches, and which kernel, are decided by the same function under the same arguments (not by `rows`:
    // every rank of the step comes to the same answer, its own slice empty or not)
    int launches = 1;
    int rc = S > 0 ? gemv_dispatch(xq, xs, Wq, sw, Ylocal, IN, rows, S, scale_dtype, st, &launches, oa) : W4A8_OK;
    if (rc != W4A8_OK) return rc;
    const bool tagged = launches == 1 && wait_limit > 0 && (size_t)S * ldY <= LL_MAX_SLOTS && mode == 0;
    if (S == 0 || rows == 0) {                       // nothing to compute: this rank still takes part in the step
        if (tagged && S > 0) {
            oa.ll = 1; oa.wait_limit = wait_limit;
            const long want = ((long)S * ldY + 255) / 256, cap = (long)sm_count() * 4;
            cudaError_t le = launch_pdl(allgather_ll_gather_kernel, dim3((unsigned)(want < cap ? want : cap)), dim3(256), 0, st, oa);
            if (le != cudaSuccess) return cuda_fail(le, "allgather_ll_gather launch");
            return launch_status("allgather_ll_gather");
        }
        allgather_publish_kernel<<<1, 32, 0, st>>>(a->desc_dev, epoch, wait_limit);
        return launch_status("allgather_publish");
    }
    rc = check_common(xq, xs, Wq, sw, Ylocal, IN, scale_dtype, "gemv_allgather");
    if (rc != W4A8_OK) return rc;
    if (!aligned(xq, 4) || !aligned(Wq, 4)) return fail(W4A8_ERR_ALIGN, "gemv_allgather: xq and Wq must be 4-byte aligned");
    rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    // One launch whose completion has to mean "Y is complete here" (wait_limit > 0) and a Y that fits a slot buffer:
    // tagged slots, no fence and no flag.  One launch and a slice small enough: the computing threads store every
    // output to every arena (W4A8_ALLGATHER=push: the last CTA copies the slice instead), and the last CTA publishes
    // the flags.  Otherwise the launches only fill the rank's own arena and the many-CTA copy kernel does the rest.
    const size_t push_total = (size_t)S * rows * sizeof(float) * (size_t)(a->world - 1);
    const bool in_kernel = tagged || (launches == 1 && push_total <= PUSH_MAX_BYTES && mode != 3);
    if (tagged) { oa.ll = 1; oa.wait_limit = wait_limit; }
    else if (in_kernel) { oa.publish = 1; oa.push = (a->world > 1 && mode == 1) ? 1 : 0; oa.local_only = mode == 1 ? 1 : 0; oa.wait_limit = wait_limit; }
    rc = gemv_dispatch(xq, xs, Wq, sw, Ylocal, IN, rows, S, scale_dtype, st, nullptr, oa);
    if (rc != W4A8_OK || in_kernel) return rc;
    return launch_scatter(a, y_offset, S, ldY, row0, rows, epoch, wait_limit, st);
}

W4A8_API int w4a8_gemv_allgather(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a, size_t y_offset,
                                 int IN, int rows, int row0, int ldY, int S, int scale_dtype, uint32_t epoch, void *stream) {
    return gemv_allgather_impl(xq, xs, Wq, sw, a, y_offset, IN, rows, row0, ldY, S, scale_dtype, epoch, 0, (cudaStream_t)stream);
}
W4A8_API int w4a8_gemv_allgather_sync(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a, size_t y_offset,
                                      int IN, int rows, int row0, int ldY, int S, int scale_dtype, uint32_t epoch, int timeout_us, void *stream) {
    return gemv_allgather_impl(xq, xs, Wq, sw, a, y_offset, IN, rows, row0, ldY, S, scale_dtype, epoch, wait_cycles(timeout_us), (cudaStream_t)stream);
}

static int gemm_allgather_impl(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a, size_t y_offset,
                               int M, int rows, int row0, int ldY, int K, int scale_dtype, uint32_t epoch, long long wait_limit, cudaStream_t st) {
    if (!a || !a->connected) return fail(W4A8_ERR_ARG, "gemm_allgather: arena not connected");
    if (M < 0 || rows < 0 || row0 < 0 || ldY < row0 + rows) return fail(W4A8_ERR_ARG, "gemm_allgather: bad shape M=%d rows=%d row0=%d ldY=%d", M, rows, row0, ldY);
    if (y_offset % 16 != 0 || y_offset + (size_t)M * ldY * sizeof(float) > a->bytes)
        return fail(W4A8_ERR_ARG, "gemm_allgather: Y[%d x %d] at offset %zu does not fit the %zu-byte arena", M, ldY, y_offset, a->bytes);
    if (K <= 0) return fail(W4A8_ERR_ARG, "gemm_allgather: K must be positive");
    if (M == 0 || rows == 0) {                       // nothing to compute: this rank still has to publish the step
        allgather_publish_kernel<<<1, 32, 0, st>>>(a->desc_dev, epoch, wait_limit);
        return launch_status("allgather_publish");
    }
    float *Ylocal = reinterpret_cast<float *>(a->base + y_offset);   // unused by the peer path; keeps the argument checks happy
    int rc = check_common(X, xs, Wq, sw, Ylocal, K, scale_dtype, "gemm_allgather");
    if (rc != W4A8_OK) return rc;
    if (!aligned(X, 16) || !aligned(Wq, 16)) return fail(W4A8_ERR_ALIGN, "gemm_allgather: X and Wq must be 16-byte aligned (TMA)");
    rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    // Two ways to get the slice to the peers: (default) the GEMM writes only its own arena and a copy kernel sends the
    // finished slice on with row-contiguous 16-byte stores; or (W4A8_GEMM_ALLGATHER=stores) the GEMM's epilogue stores
    // every tile into every arena itself, which overlaps with the compute but offers NVLink only 16-byte pieces.
    static const bool direct = [] { const char *e = getenv("W4A8_GEMM_ALLGATHER"); return e && e[0] == 's'; }();
    OutArgs oa;
    oa.peers = a->desc_dev; oa.y_off = y_offset; oa.ld = ldY; oa.col0 = row0; oa.epoch = epoch;
    oa.publish = direct ? 1 : 0; oa.local_only = direct ? 0 : 1;
    if (direct) oa.wait_limit = wait_limit;
    rc = gemm::launch_tc(X, xs, Wq, sw, Ylocal, M, rows, K, scale_dtype, 1, K / QBLK, st, oa);   // the int8 kernel carries the peer epilogue
    if (rc != W4A8_OK || direct) return rc;
    return launch_scatter(a, y_offset, M, ldY, row0, rows, epoch, wait_limit, st);
}

W4A8_API int w4a8_gemm_allgather(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a, size_t y_offset,
                                 int M, int rows, int row0, int ldY, int K, int scale_dtype, uint32_t epoch, void *stream) {
    return gemm_allgather_impl(X, xs, Wq, sw, a, y_offset, M, rows, row0, ldY, K, scale_dtype, epoch, 0, (cudaStream_t)stream);
}
W4A8_API int w4a8_gemm_allgather_sync(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a, size_t y_offset,
                                      int M, int rows, int row0, int ldY, int K, int scale_dtype, uint32_t epoch, int timeout_us, void *stream) {
    return gemm_allgather_impl(X, xs, Wq, sw, a, y_offset, M, rows, row0, ldY, K, scale_dtype, epoch, wait_cycles(timeout_us), (cudaStream_t)stream);
}

W4A8_API int w4a8_allgather_wait(w4a8_arena *a, uint32_t epoch, int timeout_us, void *stream) {
    if (!a || !a->connected) return fail(W4A8_ERR_ARG, "allgather_wait: arena not connected");
    const long long limit = wait_cycles(timeout_us);
    cudaError_t le = launch_pdl(allgather_wait_kernel, dim3(1), dim3(32), 0, (cudaStream_t)stream, (const PeerDesc *)a->desc_dev, (unsigned int)epoch, limit);
    if (le != cudaSuccess) return cuda_fail(le, "allgather_wait launch");
    return launch_status("allgather_wait");
}

W4A8_API int w4a8_arena_advance_epoch(w4a8_arena *a, uint32_t delta, void *stream) {
    if (!a || !a->connected) return fail(W4A8_ERR_ARG, "arena_advance_epoch: arena not connected");
    allgather_advance_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a->desc_dev, delta);
    return launch_status("allgather_advance");
}

// ---- routed-expert block ---------------------------------------------------------------------------------
W4A8_API int w4a8_moe_layout_for(int S, int topk, int H, int MI, int experts, w4a8_moe_layout *out) {
    if (!out || S < 0 || topk <= 0 || H <= 0 || MI <= 0 || experts <= 0 || experts > moe::MAX_EXPERTS || (long)S * topk > (1L << 24))
        return fail(W4A8_ERR_ARG, "moe_layout_for: S=%d topk=%d H=%d MI=%d experts=%d (1..%d experts)", S, topk, H, MI, experts, moe::MAX_EXPERTS);
    const moe::Layout l = moe::layout_for(S, topk, H, MI, experts);
    out->perm = l.perm; out->pos = l.pos; out->offsets = l.offsets; out->items = l.items; out->num_items = l.num_items;
    out->xq = l.xq; out->xs = l.xs; out->xq_g = l.xq_g; out->xs_g = l.xs_g; out->gu = l.gu; out->xq_h = l.xq_h; out->xs_h = l.xs_h;
    out->sout = l.sout; out->bytes = l.bytes;
    return W4A8_OK;
}

static int moe_block_impl(const float *n2, const uint8_t *gu_wq, const void *gu_sc, const uint8_t *dn_wq, const void *dn_sc,
                          const int32_t *idx, const float *dw, float *out, int S, int topk, int H, int MI, int expert_base, int experts,
                          int scale_dtype, int act, void *workspace, size_t workspace_bytes, w4a8_arena *a, size_t sout_offset,
                          uint32_t epoch, int timeout_us, int phase, cudaStream_t st, const char *who) {
    if (phase < 0 || phase > 2) return fail(W4A8_ERR_ARG, "%s: phase=%d (0 whole block, 1 compute + publish, 2 wait + combine)", who, phase);
    if (S < 0 || topk <= 0 || experts <= 0 || experts > moe::MAX_EXPERTS || expert_base < 0)
        return fail(W4A8_ERR_ARG, "%s: bad sizes S=%d topk=%d experts=%d expert_base=%d", who, S, topk, experts, expert_base);
    if (H <= 0 || MI <= 0 || H % QBLK != 0 || MI % QBLK != 0)
        return fail(W4A8_ERR_ARG, "%s: H=%d and MI=%d must be positive multiples of %d", who, H, MI, QBLK);
    if (scale_dtype < 0 || scale_dtype > 1) return fail(W4A8_ERR_ARG, "%s: scale_dtype=%d (0 fp32, 1 fp16)", who, scale_dtype);
    if (act < 0 || act > 1) return fail(W4A8_ERR_ARG, "%s: act=%d (0 SwiGLU, 1 GeGLU)", who, act);
    const long nslots = (long)S * topk;
    if (nslots > (1L << 24)) return fail(W4A8_ERR_UNSUPPORTED, "%s: at most 2^24 slots (got %ld)", who, nslots);
    if (a && !a->connected) return fail(W4A8_ERR_ARG, "%s: arena not connected", who);
    if (a && (sout_offset % 256 != 0 || sout_offset + (size_t)nslots * H * sizeof(float) > a->bytes))
        return fail(W4A8_ERR_ARG, "%s: Sout[%ld x %d] at offset %zu does not fit the %zu-byte arena", who, nslots, H, sout_offset, a->bytes);
    if (S == 0) {
        if (!a) return W4A8_OK;
        allgather_publish_kernel<<<1, 32, 0, st>>>(a->desc_dev, epoch, wait_cycles(timeout_us));   // still takes part in the step
        return launch_status("allgather_publish");
    }
    if (!n2 || !gu_wq || !gu_sc || !dn_wq || !dn_sc || !idx || !dw || !out || !workspace)
        return fail(W4A8_ERR_ARG, "%s: null pointer argument", who);
    if (!aligned(n2, 16) || !aligned(out, 16) || !aligned(gu_wq, 16) || !aligned(dn_wq, 16) || !aligned(gu_sc, 16) || !aligned(dn_sc, 16) ||
        !aligned(workspace, 256))
        return fail(W4A8_ERR_ALIGN, "%s: n2, out, the weight and scale tensors must be 16-byte aligned, the workspace 256-byte aligned", who);
    const moe::Layout l = moe::layout_for(S, topk, H, MI, experts);
    if (workspace_bytes < l.bytes) return fail(W4A8_ERR_ARG, "%s: workspace of %zu bytes, %zu needed (w4a8_moe_layout_for)", who, workspace_bytes, l.bytes);
    int rc = require_sm100();
    if (rc != W4A8_OK) return rc;
    const bool use_gemm = g_moe_policy == 2 || (g_moe_policy == 0 && nslots > moe::GEMV_MAX_SLOTS);
    if (!use_gemm && nslots > 65535) return fail(W4A8_ERR_UNSUPPORTED, "%s: the grouped GEMV takes at most 65535 slots (got %ld)", who, nslots);
    if (use_gemm && (H % 32 != 0 || MI % 32 != 0)) return fail(W4A8_ERR_UNSUPPORTED, "%s: the grouped GEMM needs H and MI multiples of 32", who);
    moe::BlockArgs b;
    b.n2 = n2; b.gu_wq = gu_wq; b.gu_sc = gu_sc; b.dn_wq = dn_wq; b.dn_sc = dn_sc; b.idx = idx; b.dw = dw; b.out = out;
    b.S = S; b.topk = topk; b.H = H; b.MI = MI; b.expert_base = expert_base; b.experts = experts; b.scale_dtype = scale_dtype; b.act = act;
    b.kernel = use_gemm ? 2 : 1;
    b.ws = static_cast<unsigned char *>(workspace);
    if (a) {
        b.peers = a->desc_dev; b.arena_base = a->base; b.sout_off = sout_offset; b.epoch = epoch; b.wait_limit = wait_cycles(timeout_us);
        b.phase = phase;
        b.world = a->world;
    }
    return moe::launch_block(b, st);
}

W4A8_API int w4a8_moe_block(const float *n2, const uint8_t *gu_wq, const void *gu_sc, const uint8_t *dn_wq, const void *dn_sc,
                            const int32_t *idx, const float *dw, float *out, int S, int topk, int H, int MI, int num_experts,
                            int scale_dtype, int act, void *workspace, size_t workspace_bytes, void *stream) {
    return moe_block_impl(n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw, out, S, topk, H, MI, 0, num_experts, scale_dtype, act, workspace,
                          workspace_bytes, nullptr, 0, 0, 0, 0, (cudaStream_t)stream, "moe_block");
}

W4A8_API int w4a8_moe_block_shard(const float *n2, const uint8_t *gu_wq, const void *gu_sc, const uint8_t *dn_wq, const void *dn_sc,
                                  const int32_t *idx, const float *dw, float *out, int S, int topk, int H, int MI, int expert_base,
                                  int experts_local, int scale_dtype, int act, void *workspace, size_t workspace_bytes, w4a8_arena *a,
                                  size_t sout_offset, uint32_t epoch, int timeout_us, int phase, void *stream) {
    if (!a) return fail(W4A8_ERR_ARG, "moe_block_shard: null arena");
    return moe_block_impl(n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw, out, S, topk, H, MI, expert_base, experts_local, scale_dtype, act,
                          workspace, workspace_bytes, a, sout_offset, epoch, timeout_us, phase, (cudaStream_t)stream, "moe_block_shard");
}
