// Drop-in for the reference's kernels/gemm_mma.cuh (launch_gemm_mma_w4a8 :129, launch_gemm_mma_w4a8_bm<BM> :119).
// The tile-height template parameter only shaped the reference's mma.sync kernel.
#pragma once
#include "w4a8_shim.h"

static inline void launch_gemm_mma_w4a8(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                        int M, int N, int K, int scale_dtype = 0, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_gemm(X, xs, Wq, sw, Y, M, N, K, scale_dtype, (void *)st), "gemm_mma_w4a8");
}
template <int BM>
static inline void launch_gemm_mma_w4a8_bm(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                           int M, int N, int K, int scale_dtype = 0, cudaStream_t st = 0) {
    launch_gemm_mma_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype, st);
}
