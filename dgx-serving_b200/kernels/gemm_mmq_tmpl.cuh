// Drop-in for the reference's kernels/gemm_mmq_tmpl.cuh: launch_gemm_mmq_tmpl<BM,BN,KT,WM,WN> (:100-105) and
// launch_gemm_mmq_w4a8_auto (:108-119).  Tile shape never changed the reference's output bits (:106-109), and the
// MMQ256 knob only chose between its tile shapes, so every variant forwards to the one tensor-core GEMM.
#pragma once
#include "gemm_mmq.cuh"

template <int BM, int BN, int KT, int WM, int WN>
static inline void launch_gemm_mmq_tmpl(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                        int M, int N, int K, int scale_dtype = 0, cudaStream_t st = 0) {
    launch_gemm_mmq_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype, st);
}
static inline void launch_gemm_mmq_w4a8_auto(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                             int M, int N, int K, int scale_dtype = 0, cudaStream_t st = 0) {
    launch_gemm_mmq_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype, st);
}
