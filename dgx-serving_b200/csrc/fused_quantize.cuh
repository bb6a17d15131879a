// Producer + quantize_x fusions: RMSNorm -> quantize and SwiGLU / GeGLU -> quantize in one kernel each.
// The reference's graphs always run norm -> quantize_x -> matmul and activation -> quantize_x -> down projection
// (models/qwen35_decode.cu:148-149, 215-218) as separate kernels with an fp32 round trip between them.  The fused
// kernels repeat the unfused element math exactly — the row sum of squares in the order of the reference's
// rmsnorm_kernel (kernels/rmsnorm.cuh:8-20: 256 threads, thread t adds elements t, t+256, ... then
// block_reduce_sum of kernels/reduce.cuh:11-24), the same rsqrtf / expf / tanhf calls and the same products — so
// xq, xs, xsum (and the optional fp32 copy of the intermediate) equal the two-kernel sequence bit for bit.
#pragma once
#include "common.cuh"

namespace w4a8 {

// One float4 of a 32-element block held by 8 consecutive lanes: block maximum and sum by three xor-shuffles, outputs
// as in quantize_x_q8_vec_kernel (d = amax / 127, q = rintf(x / d) clamped, zero block -> zeros).  Every lane of
// the warp must call it; lanes with live == false carry zeros and store nothing.
__device__ __forceinline__ void quantize_store_vec4(float4 v, long i, bool live, uint32_t *__restrict__ xq,
                                                    float *__restrict__ xs, int32_t *__restrict__ xsum) {
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float d = amax / 127.0f;
    int sum = 0;
    const uint32_t packed = amax != 0.0f ? quantize4_pack(v, d, sum) : 0u;
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    if (live) {
        xq[i] = packed;
        if ((i & 7) == 0) {
            xs[i >> 3] = d;
            if (xsum) xsum[i >> 3] = sum;
        }
    }
}

// The same for a row that stays in shared memory (the prologue of a GEMV that quantizes its own activation row): word i
// of the row -> xrow[i], the scale of block i / 8 -> xs_row[i / 8]; g_xq / g_xs (null: skipped) receive the same values.
__device__ __forceinline__ void quantize_row_vec4(float4 v, int i, bool live, uint32_t *xrow, float *xs_row,
                                                  uint32_t *__restrict__ g_xq, float *__restrict__ g_xs) {
    float amax = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    const float d = amax / 127.0f;
    int sum = 0;
    const uint32_t packed = amax != 0.0f ? quantize4_pack(v, d, sum) : 0u;
    if (live) {
        xrow[i] = packed;
        if (g_xq) g_xq[i] = packed;
        if ((i & 7) == 0) {
            xs_row[i >> 3] = d;
            if (g_xs) g_xs[i >> 3] = d;
        }
    }
}

// VARIANT 0: y = x * inv * W (launch_rmsnorm); 1: y = x * inv * (1 + W) (launch_rmsnorm_zc); 2: y = x * inv
// (launch_rmsnorm_noscale).  One CTA of 256 threads per row, as in the reference (the reduction order depends on it).
template <int VARIANT>
__global__ void __launch_bounds__(256) rmsnorm_quantize_kernel(const float *__restrict__ X, const float *__restrict__ W, float eps,
                                                               float *__restrict__ Y, uint32_t *__restrict__ xq, float *__restrict__ xs,
                                                               int32_t *__restrict__ xsum, int hh) {
    __shared__ float sh[32];
    __shared__ float inv_s;
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const size_t row = blockIdx.x;
    const float *xr = X + row * hh;
    pdl_launch_dependents();
    float ss = 0.f;
    for (int i = tid; i < hh; i += 256) { const float v = xr[i]; ss = fmaf(v, v, ss); }
    // block_reduce_sum of the reference: shfl_down tree per warp, partials through shared memory, warp 0 adds them
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_down_sync(0xffffffffu, ss, o);
    if (lane == 0) sh[wid] = ss;
    __syncthreads();
    ss = (tid < 8) ? sh[lane] : 0.0f;
    if (wid == 0) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_down_sync(0xffffffffu, ss, o);
        if (lane == 0) inv_s = rsqrtf(ss / hh + eps);
    }
    __syncthreads();
    const float inv = inv_s;
    const int n4 = hh >> 2;                      // a multiple of 8: every 8-lane group is one whole block
    const float4 *x4 = reinterpret_cast<const float4 *>(xr);
    const float4 *w4 = reinterpret_cast<const float4 *>(W);
    for (int j0 = tid; j0 - lane < n4; j0 += 256) {
        const bool live = j0 < n4;
        float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            const float4 x = x4[j0];
            if (VARIANT == 2) {
                y = make_float4(x.x * inv, x.y * inv, x.z * inv, x.w * inv);
            } else {
                const float4 w = w4[j0];
                if (VARIANT == 0) y = make_float4(x.x * inv * w.x, x.y * inv * w.y, x.z * inv * w.z, x.w * inv * w.w);
                else y = make_float4(x.x * inv * (1.0f + w.x), x.y * inv * (1.0f + w.y), x.z * inv * (1.0f + w.z), x.w * inv * (1.0f + w.w));
            }
            if (Y) reinterpret_cast<float4 *>(Y + row * hh)[j0] = y;
        }
        quantize_store_vec4(y, (long)(row * n4) + j0, live, xq, xs, xsum);
    }
}

// ACT 0: y = silu(g) * u (kernels/swiglu.cuh:5-8); 1: y = gelu_tanh(g) * u (kernels/swiglu.cuh:19-27).
template <int ACT>
__device__ __forceinline__ float glu_value(float g, float u) {
    if (ACT == 0) { const float s = g / (1.0f + expf(-g)); return s * u; }
    const float t = tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g));
    return 0.5f * g * (1.0f + t) * u;
}
template <int ACT>
__global__ void __launch_bounds__(256) glu_quantize_kernel(const float4 *__restrict__ G, const float4 *__restrict__ U, float4 *__restrict__ Y,
                                                           uint32_t *__restrict__ xq, float *__restrict__ xs, int32_t *__restrict__ xsum,
                                                           long nvec /* = S*IN/4, a multiple of 8 */, int row_vecs, long pitch_vecs) {
    // row_vecs = IN/4; rows of G and U start pitch_vecs float4s apart (== row_vecs: dense; a fused gate|up tensor
    // [S][2*IN] has pitch 2*IN/4 and U = G + IN)
    const long stride = (long)gridDim.x * blockDim.x;
    pdl_launch_dependents();
    pdl_wait();   // G and U come from the kernel before this one (a no-op unless launched for programmatic dependent launch)
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i - (threadIdx.x & 31) < nvec; i += stride) {
        const bool live = i < nvec;
        float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            const long src = pitch_vecs == row_vecs ? i : (i / row_vecs) * pitch_vecs + (i % row_vecs);
            const float4 g = G[src], u = U[src];
            y = make_float4(glu_value<ACT>(g.x, u.x), glu_value<ACT>(g.y, u.y), glu_value<ACT>(g.z, u.z), glu_value<ACT>(g.w, u.w));
            if (Y) Y[i] = y;
        }
        quantize_store_vec4(y, i, live, xq, xs, xsum);
    }
}

inline int launch_rmsnorm_quantize(const float *X, const float *W, float eps, int variant, float *Y, int8_t *xq, float *xs,
                                   int32_t *xsum, int IN, int S, cudaStream_t st) {
    uint32_t *q = reinterpret_cast<uint32_t *>(xq);
    switch (variant) {
        case 0: rmsnorm_quantize_kernel<0><<<S, 256, 0, st>>>(X, W, eps, Y, q, xs, xsum, IN); break;
        case 1: rmsnorm_quantize_kernel<1><<<S, 256, 0, st>>>(X, W, eps, Y, q, xs, xsum, IN); break;
        default: rmsnorm_quantize_kernel<2><<<S, 256, 0, st>>>(X, W, eps, Y, q, xs, xsum, IN); break;
    }
    return launch_status("rmsnorm_quantize_x_q8");
}

inline int launch_glu_quantize(const float *G, const float *U, int act, float *Y, int8_t *xq, float *xs, int32_t *xsum, int IN,
                               int S, cudaStream_t st, long pitch = 0 /* floats between rows of G / U; 0 = IN */,
                               bool pdl = false /* launch for programmatic dependent launch (inside a chain of such kernels) */) {
    const long nvec = (long)S * IN / 4;
    long want = (nvec + 255) / 256, cap = (long)sm_count() * 8;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    const float4 *g = reinterpret_cast<const float4 *>(G), *u = reinterpret_cast<const float4 *>(U);
    float4 *y = reinterpret_cast<float4 *>(Y);
    uint32_t *q = reinterpret_cast<uint32_t *>(xq);
    const long pv = (pitch > 0 ? pitch : IN) / 4;
    if (pdl) {
        cudaError_t e = act == 0 ? launch_pdl(glu_quantize_kernel<0>, dim3(grid), dim3(256), 0, st, g, u, y, q, xs, xsum, nvec, IN / 4, pv)
                                 : launch_pdl(glu_quantize_kernel<1>, dim3(grid), dim3(256), 0, st, g, u, y, q, xs, xsum, nvec, IN / 4, pv);
        if (e != cudaSuccess) return cuda_fail(e, "glu_quantize_x_q8 launch");
    } else if (act == 0) glu_quantize_kernel<0><<<grid, 256, 0, st>>>(g, u, y, q, xs, xsum, nvec, IN / 4, pv);
    else glu_quantize_kernel<1><<<grid, 256, 0, st>>>(g, u, y, q, xs, xsum, nvec, IN / 4, pv);
    return launch_status("glu_quantize_x_q8");
}

}  // namespace w4a8
