// Drop-in for the reference's kernels/gemm_mmq_raster.cuh (launch_gemm_mmq_raster_w4a8, :115-130).  raster / group
// only re-ordered the reference's CTA-to-tile map (:16-27; byte-identical outputs, tools/r25_raster_gate.cu); the
// persistent tensor-core kernel has its own M-fastest tile order.  M <= 0 or N <= 0 returns at once like the
// original (:118).
#pragma once
#include "gemm_mmq.cuh"

static inline void launch_gemm_mmq_raster_w4a8(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                               int M, int N, int K, int scale_dtype, int /*raster*/, int /*group*/,
                                               cudaStream_t st = 0) {
    if (M <= 0 || N <= 0) return;
    launch_gemm_mmq_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype, st);
}
