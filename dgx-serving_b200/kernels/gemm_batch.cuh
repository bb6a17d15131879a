// Drop-in for the W4A8 part of the reference's kernels/gemm_batch.cuh (launch_gemm_batch_w4a8, :228-231).  The
// fp32 / W4A32 batch launchers of that file are a different precision path and are not provided.
#pragma once
#include "w4a8_shim.h"

static inline void launch_gemm_batch_w4a8(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                          int IN, int OUT, int B, int scale_dtype = 0, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_gemv(xq, xs, Wq, sw, Y, IN, OUT, B, scale_dtype, (void *)st), "gemm_batch_w4a8");
}
