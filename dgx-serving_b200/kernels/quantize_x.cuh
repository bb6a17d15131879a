// Drop-in for the reference's kernels/quantize_x.cuh (launch_quantize_x_q8, :41-47).
#pragma once
#include "w4a8_shim.h"

static inline void launch_quantize_x_q8(const float *X, int8_t *xq, float *xs, int32_t *xsum, int IN, int S,
                                        cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_quantize_x_q8(X, xq, xs, xsum, IN, S, (void *)st), "quantize_x_q8");
}
