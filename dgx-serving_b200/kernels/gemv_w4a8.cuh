// Drop-in for the reference's kernels/gemv_w4a8.cuh: the plain, mlp<U>, mlp_auto, SB, g4 and SB-g4 launchers
// (:93, :102, :155, :168, :316, :337).  All of them compute the same product, so all forward to w4a8_gemv; the
// unroll / prefetch / unpack knobs (MLP_U, G4_GEMV_U, G4_GEMV_PF, G4_GEMV_PERM) only scheduled the reference's
// kernels and have nothing to select here.  The xsum argument was already unused in the reference (:23-25).
#pragma once
#include "w4a8_shim.h"
#include "qscale.cuh"
#include "reduce.cuh"

#ifdef __CUDACC__
// Device helper other files of the reference borrow from its header (kernels/gemv_w4a8.cuh:16-21; tools/probe_*.cu):
// two packed bytes = four 4-bit codes (low nibble first) -> four signed bytes (code - 8), the dp4a operand.
static __device__ __forceinline__ int w4a8_pk(int lo_byte, int hi_byte) {
    const unsigned v = (unsigned)(lo_byte & 0x0F) | ((unsigned)(lo_byte & 0xF0) << 4) | ((unsigned)(hi_byte & 0x0F) << 16) |
                       ((unsigned)(hi_byte & 0xF0) << 20);       // one code per byte
    return (int)__vsub4(v, 0x08080808u);                         // minus 8 in every byte
}
#endif

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

// Two matrices against one quantized input (gate + up, k + v) in one call: one kernel launch for a single decode row
// (no counterpart in the reference; same bits as two launch_gemv_w4a8 calls).
static inline void launch_gemv_w4a8_pair(const int8_t *xq, const float *xs, const uint8_t *Wq1, const void *sc1, float *Y1, int OUT1,
                                         const uint8_t *Wq2, const void *sc2, float *Y2, int OUT2, int IN, int S, int scale_dtype = 0,
                                         cudaStream_t st = 0) {
    const uint8_t *wq[2] = {Wq1, Wq2};
    const void *sc[2] = {sc1, sc2};
    float *y[2] = {Y1, Y2};
    const int out[2] = {OUT1, OUT2};
    w4a8_shim_check(w4a8_gemv_multi(xq, xs, 2, wq, sc, y, out, IN, S, scale_dtype, (void *)st), "gemv_w4a8_pair");
}
