// Drop-in for the reference's kernels/quantize_x.cuh (launch_quantize_x_q8, :41-47).
#pragma once
#include "w4a8_shim.h"

static inline void launch_quantize_x_q8(const float *X, int8_t *xq, float *xs, int32_t *xsum, int IN, int S,
                                        cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_quantize_x_q8(X, xq, xs, xsum, IN, S, (void *)st), "quantize_x_q8");
}

// Fused forms for the graphs' norm -> quantize and activation -> quantize pairs (no counterpart in the reference;
// each gives the bits of the reference's two launchers run one after the other).  `norm` / `act_out` may be nullptr
// when nothing else reads the fp32 intermediate.
//   launch_rmsnorm_zc(x, w, norm, S, H, eps); launch_quantize_x_q8(norm, xq, xs, xsum, H, S);
//     -> launch_rmsnorm_zc_quantize_x_q8(x, w, norm, xq, xs, xsum, S, H, eps);
//   launch_swiglu(g, u, act, S*FFN); launch_quantize_x_q8(act, xq, xs, xsum, FFN, S);
//     -> launch_swiglu_quantize_x_q8(g, u, act, xq, xs, xsum, FFN, S);
static inline void launch_rmsnorm_quantize_x_q8(const float *X, const float *W, float *norm, int8_t *xq, float *xs, int32_t *xsum,
                                                int rows, int hh, float eps, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_rmsnorm_quantize_x_q8(X, W, eps, 0, norm, xq, xs, xsum, hh, rows, (void *)st), "rmsnorm_quantize_x_q8");
}
static inline void launch_rmsnorm_zc_quantize_x_q8(const float *X, const float *W, float *norm, int8_t *xq, float *xs, int32_t *xsum,
                                                   int rows, int hh, float eps, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_rmsnorm_quantize_x_q8(X, W, eps, 1, norm, xq, xs, xsum, hh, rows, (void *)st), "rmsnorm_zc_quantize_x_q8");
}
static inline void launch_rmsnorm_noscale_quantize_x_q8(const float *X, float *norm, int8_t *xq, float *xs, int32_t *xsum, int rows,
                                                        int hh, float eps, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_rmsnorm_quantize_x_q8(X, nullptr, eps, 2, norm, xq, xs, xsum, hh, rows, (void *)st), "rmsnorm_noscale_quantize_x_q8");
}
static inline void launch_swiglu_quantize_x_q8(const float *g, const float *u, float *act_out, int8_t *xq, float *xs, int32_t *xsum,
                                               int IN, int S, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_glu_quantize_x_q8(g, u, 0, act_out, xq, xs, xsum, IN, S, (void *)st), "swiglu_quantize_x_q8");
}
static inline void launch_geglu_quantize_x_q8(const float *g, const float *u, float *act_out, int8_t *xq, float *xs, int32_t *xsum,
                                              int IN, int S, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_glu_quantize_x_q8(g, u, 1, act_out, xq, xs, xsum, IN, S, (void *)st), "geglu_quantize_x_q8");
}
