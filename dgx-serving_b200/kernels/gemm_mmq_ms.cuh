// Drop-in for the reference's kernels/gemm_mmq_ms.cuh (multi-stage cp.async proof of concept, tools only): same
// product, so launch_gemm_mmq_ms<...> forwards to the tensor-core GEMM.
#pragma once
#include "gemm_mmq.cuh"

template <int BM, int BN, int KT, int WM, int WN, int STAGES>
static inline void launch_gemm_mmq_ms(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                      int M, int N, int K, int scale_dtype = 0, cudaStream_t st = 0) {
    launch_gemm_mmq_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype, st);
}
