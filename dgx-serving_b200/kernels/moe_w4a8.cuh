// W4A8 form of the reference's device-fused routed-expert path.  The call site is models/moe_block.cuh:45-52: after
// launch_router_topk has left the expert ids (didx) and router weights (dw) of the S*K slots on the device, the
// reference enqueues launch_moe_fused_gu / _swiglu / _down / _reduce (kernels/moe_fused.cuh:78-103) on fp32
// activations.  launch_moe_w4a8_block takes the same tensors and does the same four steps with the expert products in
// W4A8 (activations quantized per 32-element block), in one call:
//
//     if (g_fused) {
//         launch_moe_w4a8_block(n2, L.experts_gate_up.wq, L.experts_gate_up.sc, L.experts_down.wq, L.experts_down.sc,
//                               didx, dw, out, S, H, MI, E, K, sdtype);
//     }
//
// Like the reference's block (moe_grow, models/moe_block.cuh:24-29) it keeps its scratch in a grow-only file-scope
// static that is allocated on first use — so, like the original, the first call for a given size must not be made
// under stream capture — and `out` is overwritten, not accumulated into (the reduce at kernels/moe_fused.cuh:69-76
// does the same), so the shared-expert part that follows (models/moe_block.cuh:69-79) stays as it is.
#pragma once
#include "w4a8_shim.h"

static void *g_w4a8_shim_moe_ws = nullptr;
static size_t g_w4a8_shim_moe_cap = 0;
static inline void launch_moe_w4a8_block(const float *n2, const uint8_t *gu_wq, const void *gu_sc, const uint8_t *dn_wq,
                                         const void *dn_sc, const int *didx, const float *dw, float *out, int S, int H, int MI,
                                         int E, int K, int sdtype = 0, cudaStream_t st = 0) {
    w4a8_moe_layout lay;
    w4a8_shim_check(w4a8_moe_layout_for(S, K, H, MI, E, &lay), "moe_layout_for");
    if (lay.bytes > g_w4a8_shim_moe_cap) {
        if (g_w4a8_shim_moe_ws) cudaFree(g_w4a8_shim_moe_ws);
        if (cudaMalloc(&g_w4a8_shim_moe_ws, lay.bytes) != cudaSuccess) { fprintf(stderr, "w4a8 shim: MoE workspace\n"); exit(1); }
        g_w4a8_shim_moe_cap = lay.bytes;
    }
    w4a8_shim_check(w4a8_moe_block(n2, gu_wq, gu_sc, dn_wq, dn_sc, (const int32_t *)didx, dw, out, S, K, H, MI, E, sdtype, /*act=*/0,
                                   g_w4a8_shim_moe_ws, g_w4a8_shim_moe_cap, (void *)st), "moe_block");
}
