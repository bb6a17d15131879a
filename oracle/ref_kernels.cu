// Thin C-ABI wrapper around the reference's OWN kernel headers, compiled from where they lie
// (-I<reference root>); no reference source is copied here.  TEST / BASELINE INFRASTRUCTURE ONLY:
// the result (oracle/_ref/libref_kernels.so) is the reference's GPU code rebuilt for sm_100a, used
// by the GPU parity tests as the bit-exact checker and by bench.py as the timed "reference kernels
// on B200" baseline.  The shipped library never loads it.
#include <cstdint>
#include <cuda_runtime.h>
#include "kernels/quantize_x.cuh"
#include "kernels/rmsnorm.cuh"
#include "kernels/swiglu.cuh"
#include "kernels/gemv_w4a8.cuh"
#include "kernels/gemm_batch.cuh"
#include "kernels/gemm_mma.cuh"
#include "kernels/gemm_mmq.cuh"
#include "kernels/gemm_mmq_tmpl.cuh"
#include "kernels/gemm_mmq_raster.cuh"
#include "kernels/moe_fused.cuh"

#define REF_API extern "C" __attribute__((visibility("default")))
static inline int ref_status() { return (int)cudaPeekAtLastError(); }

REF_API int ref_quantize_x_q8(const float *X, int8_t *xq, float *xs, int32_t *xsum, int IN, int S, void *st) {
    launch_quantize_x_q8(X, xq, xs, xsum, IN, S, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemv_w4a8(const int8_t *xq, const float *xs, const int32_t *xsum, const uint8_t *Wq, const void *sw,
                          float *Y, int IN, int OUT, int S, int sd, void *st) {
    launch_gemv_w4a8(xq, xs, xsum, Wq, sw, Y, IN, OUT, S, sd, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemv_w4a8_mlp2(const int8_t *xq, const float *xs, const int32_t *xsum, const uint8_t *Wq, const void *sw,
                               float *Y, int IN, int OUT, int S, int sd, void *st) {
    launch_gemv_w4a8_mlp<2>(xq, xs, xsum, Wq, sw, Y, IN, OUT, S, sd, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemv_w4a8_sb(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw,
                             float *Y, int IN, int OUT, int S, int sd, void *st) {
    launch_gemv_w4a8_sb(xq, xs, Wq, sw, Y, IN, OUT, S, sd, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemm_batch_w4a8(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw,
                                float *Y, int IN, int OUT, int B, int sd, void *st) {
    launch_gemm_batch_w4a8(xq, xs, Wq, sw, Y, IN, OUT, B, sd, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemm_mma_w4a8(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw,
                              float *Y, int M, int N, int K, int sd, void *st) {
    launch_gemm_mma_w4a8(X, xs, Wq, sw, Y, M, N, K, sd, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemm_mmq_w4a8(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw,
                              float *Y, int M, int N, int K, int sd, void *st) {
    launch_gemm_mmq_w4a8(X, xs, Wq, sw, Y, M, N, K, sd, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemm_mmq_256x64(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw,
                                float *Y, int M, int N, int K, int sd, void *st) {
    launch_gemm_mmq_tmpl<256, 64, 64, 4, 2>(X, xs, Wq, sw, Y, M, N, K, sd, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemm_mmq_raster_w4a8(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw,
                                     float *Y, int M, int N, int K, int sd, int raster, int group, void *st) {
    launch_gemm_mmq_raster_w4a8(X, xs, Wq, sw, Y, M, N, K, sd, raster, group, (cudaStream_t)st); return ref_status();
}
REF_API int ref_gemm_bm16_splitk(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw,
                                 float *Y, int M, int N, int K, int sd, void *st) {
    launch_gemm_bm16_splitk(X, xs, Wq, sw, Y, M, N, K, sd, (cudaStream_t)st); return ref_status();
}

// The producers of quantize_x in the graphs (models/qwen35_decode.cu:148-149, 215-218), for the fused entries' parity.
REF_API int ref_rmsnorm(const float *X, const float *W, float *Y, int rows, int hh, float eps, int variant, void *st) {
    if (variant == 0) launch_rmsnorm(X, W, Y, rows, hh, eps, (cudaStream_t)st);
    else if (variant == 1) launch_rmsnorm_zc(X, W, Y, rows, hh, eps, (cudaStream_t)st);
    else launch_rmsnorm_noscale(X, Y, rows, hh, eps, (cudaStream_t)st);
    return ref_status();
}
REF_API int ref_glu(const float *g, const float *u, float *Y, long n, int act, void *st) {
    if (act == 0) launch_swiglu(g, u, Y, (size_t)n, (cudaStream_t)st);
    else launch_geglu(g, u, Y, (size_t)n, (cudaStream_t)st);
    return ref_status();
}

// The reference's device-fused routed-expert path exactly as models/moe_block.cuh:45-52 enqueues it (W4A32: fp32
// activations against the packed int4 experts): grouped gate_up, swiglu, grouped down, fixed-order reduce.
// fgu [nslot][2*MI], fhid [nslot][MI], fsout [nslot][H] are the caller's scratch.
REF_API int ref_moe_fused_block(const float *n2, const uint8_t *gu_wq, const void *gu_sc, const uint8_t *dn_wq, const void *dn_sc,
                                const int *didx, const float *dw, float *fgu, float *fhid, float *fsout, float *out, int S, int H,
                                int MI, int K, int sd, void *st) {
    const long nslot = (long)S * K;
    const long gu_w = 2L * MI * H, dn_w = (long)H * MI;
    launch_moe_fused_gu(n2, gu_wq, gu_sc, didx, fgu, H, 2 * MI, K, nslot, gu_w, sd, (cudaStream_t)st);
    launch_moe_fused_swiglu(fgu, fhid, MI, nslot, (cudaStream_t)st);
    launch_moe_fused_down(fhid, dn_wq, dn_sc, didx, dw, fsout, MI, H, K, nslot, dn_w, sd, (cudaStream_t)st);
    launch_moe_fused_reduce(fsout, out, H, K, S, (cudaStream_t)st);
    return ref_status();
}
