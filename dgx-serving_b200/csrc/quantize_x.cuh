// Activation quantization, fp32 row -> int8 + per-32-block scale (+ block sums).
// Semantics: reference kernels/quantize_x.cuh:22-39 (d = amax/127.0f, q = rintf(x/d), clamp +-127,
// all-zero block -> q = 0 and d = 0).  HBM-bound: 5.25 bytes moved per element.
#pragma once
#include "common.cuh"

namespace w4a8 {

// Eight threads own one 32-element block: each loads a float4 (16 B), the block maximum and the block
// sum are formed with three xor-shuffles inside the 8-lane group, each thread stores its 4 int8 as one
// 32-bit word.  A warp therefore reads 512 contiguous bytes and writes 128.  UNROLL independent vectors
// per thread are loaded before any is used, to keep enough bytes in flight per SM.
template <int UNROLL>
__global__ void __launch_bounds__(256) quantize_x_q8_vec_kernel(const float4 *__restrict__ X, uint32_t *__restrict__ xq,
                                                                float *__restrict__ xs, int32_t *__restrict__ xsum,
                                                                long nvec /* = S*IN/4, a multiple of 8 */) {
    const long stride = (long)gridDim.x * blockDim.x;
    long i0 = (long)blockIdx.x * blockDim.x + threadIdx.x;
    // Lets a following kernel that was launched for programmatic dependent launch (the GEMV) become resident and
    // start streaming its weights while this kernel runs; it still waits for this kernel's completion before it
    // reads xq / xs.
    pdl_launch_dependents();
    // nvec is a multiple of 8 and i0 - lane is a multiple of 32, so the 8-lane groups are either fully
    // inside or fully outside; shuffles use the full mask with out-of-range lanes carrying zeros.
    for (; i0 - (threadIdx.x & 31) < nvec; i0 += stride * UNROLL) {
        float4 v[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            long i = i0 + u * stride;
            v[u] = (i < nvec) ? __ldcs(X + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; u++) {
            long i = i0 + u * stride;
            float amax = fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w)));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float d = amax / 127.0f;
            int sum = 0;
            const uint32_t packed = amax != 0.0f ? quantize4_pack(v[u], d, sum) : 0u;
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            if (i < nvec) {
                xq[i] = packed;
                if ((i & 7) == 0) {
                    xs[i >> 3] = d;
                    if (xsum) xsum[i >> 3] = sum;
                }
            }
        }
    }
}

// Same arithmetic with one lane per element (one warp per block), for pointers that are only 4-byte
// aligned: the reference's launcher accepts those.
__global__ void __launch_bounds__(256) quantize_x_q8_scalar_kernel(const float *__restrict__ X, int8_t *__restrict__ xq,
                                                                   float *__restrict__ xs, int32_t *__restrict__ xsum,
                                                                   long nblk) {
    const int lane = threadIdx.x & 31;
    const long wstride = ((long)gridDim.x * blockDim.x) >> 5;
    for (long b = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < nblk; b += wstride) {
        const float x = X[b * QBLK + lane];
        float amax = fabsf(x);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const float d = amax / 127.0f;
        int q = (amax == 0.0f) ? 0 : (int)rintf(x / d);
        q = max(-127, min(127, q));
        int sum = q;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        xq[b * QBLK + lane] = (int8_t)q;
        if (lane == 0) {
            xs[b] = d;
            if (xsum) xsum[b] = sum;
        }
    }
}

inline int launch_quantize_x(const float *X, int8_t *xq, float *xs, int32_t *xsum, int IN, int S, cudaStream_t st) {
    if (S == 0 || IN == 0) return W4A8_OK;
    const long nblk = (long)S * (IN / QBLK);
    const int sms = sm_count();
    if (aligned(X, 16) && aligned(xq, 4)) {
        const long nvec = nblk * 8;
        constexpr int U = 4;
        long want = (nvec + 256L * U - 1) / (256L * U);
        long cap = (long)sms * 8;  // 8 CTAs of 256 threads fill an SM
        unsigned grid = (unsigned)(want < cap ? want : cap);
        quantize_x_q8_vec_kernel<U><<<grid, 256, 0, st>>>(reinterpret_cast<const float4 *>(X),
                                                          reinterpret_cast<uint32_t *>(xq), xs, xsum, nvec);
    } else {
        long want = (nblk + 7) / 8;
        long cap = (long)sms * 8;
        unsigned grid = (unsigned)(want < cap ? want : cap);
        quantize_x_q8_scalar_kernel<<<grid, 256, 0, st>>>(X, xq, xs, xsum, nblk);
    }
    return launch_status("quantize_x_q8");
}

}  // namespace w4a8
