// Drop-in for the reference's kernels/gemv_w4a8.cuh: the plain, mlp<U>, mlp_auto, SB, g4 and SB-g4 launchers
// (:93, :102, :155, :168, :316, :337).  All of them compute the same product, so all forward to w4a8_gemv; the
// unroll / prefetch / unpack knobs (MLP_U, G4_GEMV_U, G4_GEMV_PF, G4_GEMV_PERM) only scheduled the reference's
// kernels and have nothing to select here.  The xsum argument was already unused in the reference (:23-25).
#pragma once
#include "w4a8_shim.h"
#include "qscale.cuh"
#include "reduce.cuh"

static inline void launch_gemv_w4a8(const int8_t *xq, const float *xs, const int32_t * /*xsum*/, const uint8_t *Wq,
                                    const void *sw, float *Y, int IN, int OUT, int S, int scale_dtype = 0,
                                    cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_gemv(xq, xs, Wq, sw, Y, IN, OUT, S, scale_dtype, (void *)st), "gemv_w4a8");
}
template <int U>
static inline void launch_gemv_w4a8_mlp(const int8_t *xq, const float *xs, const int32_t *xsum, const uint8_t *Wq,
                                        const void *sw, float *Y, int IN, int OUT, int S, int scale_dtype = 0,
                                        cudaStream_t st = 0) {
    launch_gemv_w4a8(xq, xs, xsum, Wq, sw, Y, IN, OUT, S, scale_dtype, st);
}
static inline void launch_gemv_w4a8_mlp_auto(const int8_t *xq, const float *xs, const int32_t *xsum, const uint8_t *Wq,
                                             const void *sw, float *Y, int IN, int OUT, int S, int scale_dtype = 0,
                                             cudaStream_t st = 0) {
    launch_gemv_w4a8(xq, xs, xsum, Wq, sw, Y, IN, OUT, S, scale_dtype, st);
}
static inline void launch_gemv_w4a8_g4(const int8_t *xq, const float *xs, const int32_t *xsum, const uint8_t *Wq,
                                       const void *sw, float *Y, int IN, int OUT, int S, int scale_dtype = 0,
                                       cudaStream_t st = 0) {
    launch_gemv_w4a8(xq, xs, xsum, Wq, sw, Y, IN, OUT, S, scale_dtype, st);
}
static inline void launch_gemv_w4a8_sb(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                       int IN, int OUT, int S, int scale_dtype = 0, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_gemv(xq, xs, Wq, sw, Y, IN, OUT, S, scale_dtype, (void *)st), "gemv_w4a8_sb");
}
static inline void launch_gemv_w4a8_sb_g4(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                          int IN, int OUT, int S, int scale_dtype = 0, cudaStream_t st = 0) {
    launch_gemv_w4a8_sb(xq, xs, Wq, sw, Y, IN, OUT, S, scale_dtype, st);
}
