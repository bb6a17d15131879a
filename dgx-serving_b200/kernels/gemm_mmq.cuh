// Drop-in for the reference's kernels/gemm_mmq.cuh: launch_gemm_mmq_w4a8 (:230), launch_gemm_mmq_w4a8_kt<KT> (:222)
// and launch_gemm_bm16_splitk (:205-219).  The reference's split-K launcher keeps a grow-only workspace in a
// file-scope static that it cudaMalloc's inside the launch (:206,:215); this shim keeps the same contract (static,
// grow-only, allocated on first use and therefore, like the original, not to be first-called under stream capture)
// and hands the buffer to w4a8_gemm_splitk, whose ABI leaves ownership with the caller.
#pragma once
#include "w4a8_shim.h"
#include "gemv_w4a8.cuh"

#ifdef __CUDACC__
// Device helper the reference's other GEMM headers and tools borrow (kernels/gemm_mmq.cuh:25-28): the low 16 bits of
// h = four 4-bit codes (low nibble first) -> four signed bytes (code - 8), an mma.sync s8 operand register.
__device__ __forceinline__ int mmq_unpack4v(unsigned h) {
    const unsigned v = (h & 0x000Fu) | ((h & 0x00F0u) << 4) | ((h & 0x0F00u) << 8) | ((h & 0xF000u) << 12);
    return (int)__vsub4(v, 0x08080808u);
}
#endif

static inline void launch_gemm_mmq_w4a8(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                        int M, int N, int K, int scale_dtype = 0, cudaStream_t st = 0) {
    w4a8_shim_check(w4a8_gemm(X, xs, Wq, sw, Y, M, N, K, scale_dtype, (void *)st), "gemm_mmq_w4a8");
}
template <int KT>
static inline void launch_gemm_mmq_w4a8_kt(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                           int M, int N, int K, int scale_dtype = 0, cudaStream_t st = 0) {
    launch_gemm_mmq_w4a8(X, xs, Wq, sw, Y, M, N, K, scale_dtype, st);
}
static void *g_w4a8_shim_skwksp = nullptr;
static size_t g_w4a8_shim_skwcap = 0;
static inline void launch_gemm_bm16_splitk(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                                           int M, int N, int K, int scale_dtype = 0, cudaStream_t st = 0) {
    // the reference's SPLITK knob, read once (kernels/gemm_mmq.cuh:210; registry row runtime/knobs.h:91-92: int, 0.. , 0 = automatic)
    static const int splitk = [] { const char *v = w4a8_shim_knob("SPLITK"); const int k = v ? atoi(v) : 0; return k > 0 ? k : 0; }();
    const size_t need = w4a8_gemm_splitk_workspace_bytes(M, N, K, splitk);
    if (need > g_w4a8_shim_skwcap) {
        if (g_w4a8_shim_skwksp) cudaFree(g_w4a8_shim_skwksp);
        if (cudaMalloc(&g_w4a8_shim_skwksp, need) != cudaSuccess) { fprintf(stderr, "w4a8 shim: split-K workspace\n"); exit(1); }
        g_w4a8_shim_skwcap = need;
    }
    w4a8_shim_check(w4a8_gemm_splitk(X, xs, Wq, sw, Y, M, N, K, scale_dtype, splitk, g_w4a8_shim_skwksp, g_w4a8_shim_skwcap,
                                     (void *)st), "gemm_bm16_splitk");
}
