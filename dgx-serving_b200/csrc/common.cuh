// Shared host/device helpers of the W4A8 library (sm_100a only).
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include "../../include/w4a8_b200.h"

#define W4A8_API extern "C" __attribute__((visibility("default")))

namespace w4a8 {

constexpr int QBLK = W4A8_QBLK;

// ---- host-side error text ----------------------------------------------------------------------
char *err_buf();  // thread-local 512-byte buffer (api.cu)
inline int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(err_buf(), 512, fmt, ap);
    va_end(ap);
    return code;
}
inline int cuda_fail(cudaError_t e, const char *what) {
    return fail(W4A8_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}
// After a kernel launch: reports launch-configuration errors without synchronising.
inline int launch_status(const char *what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) { cudaGetLastError(); return cuda_fail(e, what); }
    return W4A8_OK;
}
inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// A value per CUDA device, selected by the current device: launch-side caches of per-device facts (function
// attributes such as the dynamic shared-memory opt-in, occupancy answers) must not leak from one GPU to the next in
// a process that drives several.
template <typename T>
struct PerDevice {
    static constexpr int MAX_DEV = 64;
    T v[MAX_DEV] = {};
    T &get() {
        int d = 0;
        if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MAX_DEV) d = 0;
        return v[d];
    }
};

// Number of SMs of the current device (148 on B200), cached per device.
int sm_count();
// W4A8_OK if the current device is compute capability 10.x, else W4A8_ERR_UNSUPPORTED.
int require_sm100();

// ---- programmatic dependent launch ---------------------------------------------------------------
// Kernels that only READ data no earlier kernel of the stream writes (the weights) before they touch anything
// else are launched with the programmatic-stream-serialization attribute: their CTAs may become resident while
// the previous kernel of the stream is still draining, issue their first weight loads, and then block in
// pdl_wait() until that kernel has completed and its writes are visible.  That hides the launch gap and the
// ramp-up of a 10-microsecond kernel behind the tail of its predecessor.  Without the attribute both
// instructions do nothing.  W4A8_PDL=0 in the environment disables the attribute (plain stream order).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
bool pdl_enabled();   // w4a8_b200.cu

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- device-side error word (set when a bounded wait runs out) ---------------------------------
__device__ unsigned int g_dev_error = 0u;  // one translation unit: w4a8_b200.cu includes every kernel file
__device__ __forceinline__ void dev_set_error(unsigned int code) { atomicCAS(&g_dev_error, 0u, code); }

#ifdef __CUDACC__
// ---- weight scale read: float, or __half widened (reference: kernels/qscale.cuh:5-6) -----------
__device__ __forceinline__ float sval(float x) { return x; }
__device__ __forceinline__ float sval(__half x) { return __half2float(x); }

// ---- int4 -> int8 expansion ------------------------------------------------------------------
// One 32-bit word of packed weights holds 8 nibbles: byte j = element 2j (low) and 2j+1 (high).
// Instead of (nibble - 8) the expansion produces 16*(nibble - 8) in each int8 byte: XOR with 8
// turns the nibble into the 4-bit two's-complement code of (nibble - 8), and a nibble sitting in
// the HIGH half of a byte with a zero low half is that value times 16.  Integer dot products are
// then 16x the true ones (still exact: |16*D| <= 520,192) and the factor 1/16 is folded into the
// fp32 scale, where it is exact.  Cost: 3 logic ops per 8 weights, no per-byte subtraction.
//   even: bytes = 16*w[0], 16*w[2], 16*w[4], 16*w[6]   (the word's low nibbles)
//   odd : bytes = 16*w[1], 16*w[3], 16*w[5], 16*w[7]   (the word's high nibbles)
__device__ __forceinline__ void unpack8_x16(uint32_t w, uint32_t &even, uint32_t &odd) {
    odd = (w & 0xF0F0F0F0u) ^ 0x80808080u;
    even = ((w << 4) & 0xF0F0F0F0u) ^ 0x80808080u;
}
// The same 8 weights in element order (for tensor-core operands): lo = 16*w[0..3], hi = 16*w[4..7].
__device__ __forceinline__ void unpack8_x16_seq(uint32_t w, uint32_t &lo, uint32_t &hi) {
    uint32_t even, odd;
    unpack8_x16(w, even, odd);
    lo = __byte_perm(even, odd, 0x5140);  // e0 o0 e1 o1
    hi = __byte_perm(even, odd, 0x7362);  // e2 o2 e3 o3
}
// Four quantized activations of one float4: q = rintf(x / d) clamped to +-127 (kernels/quantize_x.cuh:36-37), packed into
// one word (byte i = q_i), and their sum.  The quotient is at most 127 * (1 + 2^-23) in magnitude because |x| <= amax
// and d = amax / 127 rounded, so the clamp never changes a finite value: one cvt.rni.sat.s8.f32 per element does
// round-to-nearest-even, the conversion and the saturation (a NaN quotient — amax infinite — gives 0 either way).
__device__ __forceinline__ uint32_t quantize4_pack(float4 v, float d, int &sum) {
    int q0, q1, q2, q3;
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q0) : "f"(v.x / d));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q1) : "f"(v.y / d));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q2) : "f"(v.z / d));
    asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(q3) : "f"(v.w / d));
    const uint32_t lo = __byte_perm((uint32_t)q0, (uint32_t)q1, 0x0040), hi = __byte_perm((uint32_t)q2, (uint32_t)q3, 0x0040);
    const uint32_t w = __byte_perm(lo, hi, 0x5410);
    sum = __dp4a((int)w, 0x01010101, 0);
    return w;
}
// Activation bytes x[0..7] (two words) split the same way: even = x0 x2 x4 x6, odd = x1 x3 x5 x7.
__device__ __forceinline__ void split_even_odd(uint32_t x0, uint32_t x1, uint32_t &even, uint32_t &odd) {
    even = __byte_perm(x0, x1, 0x6420);
    odd = __byte_perm(x0, x1, 0x7531);
}
#endif

}  // namespace w4a8
