// W4A8 decode GEMV on the warp-level int8 tensor path (mma.sync m16n8k32) for 1..16 activation rows.
// Same product as csrc/gemv_w4a8.cuh (the reference's kernels/gemv_w4a8.cuh:119-151 SB kernel and
// kernels/gemm_batch.cuh:187-213): the weights are streamed exactly once for all S rows.  The difference is
// where the integer work runs: with more than a couple of activation rows the dp4a formulation needs more
// issue slots than an SM has at HBM speed, so here 16 weight rows x one 32-element group x 8 activation rows
// is ONE tensor instruction, and what is left for the CUDA cores is the scale-and-accumulate per (row, m, group).
//
// fp32 evaluation order: per (m, n) one accumulator, groups ascending, t = (float)D * xs[m,b] (rounded),
// acc = fma(t, sw[n,b], acc) — the order of the reference's MMQ kernels (kernels/gemm_mmq.cuh:104-105) and of
// this library's tensor-core GEMM, so every entry point that lands here agrees with them bit for bit, for any S.
//
// Data flow per warp (no CTA-wide synchronisation after the prologue):
//   cp.async (16 B per lane, L1 bypass) brings a step = 16 weight rows x 4 groups (1 KB) plus their 16 x 4 scales
//   into a warp-private ring of STAGES slots; the slot layout is [row][4 x 16 B] with the 16-byte pieces XOR-swizzled
//   so that ldmatrix reads are bank-conflict free;
//   ldmatrix.x4 hands lane (g = lane/4, t = lane%4) the 4 bytes at offset 4t of rows g and g+8 of two groups: exactly
//   the packed word whose even / odd nibbles (unpack8_x16: 16*(w-8), three logic ops) are the A-fragment registers;
//   the activations, staged once per CTA and pre-split into the matching even / odd byte order, are the B fragment;
//   D[16 x 8] int32 = 16 * group dots; the factor 1/16 is folded (exactly) into the staged activation scales.
#pragma once
#include "common.cuh"
#include "gemv_w4a8.cuh"

namespace w4a8 {
namespace gemv_mma {

#ifndef W4A8_MMA_WARPS
#define W4A8_MMA_WARPS 8
#endif
constexpr int WARPS = W4A8_MMA_WARPS;
#ifndef W4A8_GEMV_RELAY
#define W4A8_GEMV_RELAY 1
#endif
constexpr bool RELAY = W4A8_GEMV_RELAY != 0;
// A step = 16 weight rows x GS groups (GS * 16 B contiguous per row) plus the 16 x GS scales (slot sized for fp32).
__host__ __device__ constexpr int step_w(int GS) { return 16 * GS * 16; }
__host__ __device__ constexpr int step_bytes(int GS) { return 16 * GS * 16 + 16 * GS * 4; }

__device__ __forceinline__ void cp_async16_cg(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async16_ca(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async8_ca(uint32_t dst, const void *src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr) : "memory");
}
// D(16x8, s32) = A(16x32, s8, row) * B(32x8, s8, col); accumulators start at zero.
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
                 : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// Shared-memory plan (bytes), all offsets multiples of 16:
//   xq'  : S rows x pitch2 uint2      (pitch2 = 4*nb + 4: rows 4 uint2 apart modulo 16 -> conflict-free LDS.64)
//   xs'  : nb x (8*MH) floats          ([group][m], already multiplied by 1/16)
//   ring : WARPS x STAGES x step_bytes(GS)
__host__ __device__ inline int pitch2_of(int nb) { return 4 * nb + 4; }
// Only the S rows that exist are staged (rows S..8*MH-1 of the MMA's B operand are zeros made in registers), so a
// single-row decode call keeps its footprint small enough for the next kernel's CTA to become resident beside it.
__host__ __device__ inline size_t xq_bytes(int S, int nb) { return (size_t)S * pitch2_of(nb) * 8; }
__host__ __device__ inline size_t act_bytes(int MH, int S, int nb) { return xq_bytes(S, nb) + (size_t)nb * 8 * MH * 4; }
__host__ __device__ inline size_t smem_bytes(int MH, int S, int nb, int GS, int STAGES) {
    return act_bytes(MH, S, nb) + (size_t)WARPS * STAGES * step_bytes(GS);
}
// 16-byte piece j of row r of a slot sits at piece position j ^ swz(r): with it the eight rows of an ldmatrix
// matrix hit eight different 16-byte bank groups (row pitch GS*16 B is a multiple of 128 B for GS >= 8).
__device__ __forceinline__ int swz(int r, int GS) { return GS >= 8 ? (r & 7) : ((r >> 1) & 3); }

template <int MH, int GS, int STAGES, typename ST, bool PEER>
__global__ void __launch_bounds__(WARPS * 32, 1) gemv_w4a8_mma_kernel(
    const int8_t *__restrict__ xq, const float *__restrict__ xs, const uint8_t *__restrict__ Wq,
    const ST *__restrict__ sw, float *__restrict__ Y, int IN, int OUT, int S, OutArgs oa) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int STEP_W = step_w(GS), STEP_BYTES = step_bytes(GS);
    const int nb = IN / QBLK, nsteps = nb / GS;       // nb % GS == 0 is a launch precondition
    const int pitch2 = pitch2_of(nb);
    uint2 *xqp = reinterpret_cast<uint2 *>(smem);
    float *sxs = reinterpret_cast<float *>(smem + xq_bytes(S, nb));
    unsigned char *ring0 = smem + act_bytes(MH, S, nb);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    // 8-row units [u0, u1) of this CTA; a warp walks them two at a time (one 16-row MMA tile)
    const int units = (OUT + 7) / 8;
    const int u0 = (int)(((long)units * blockIdx.x) / gridDim.x), u1 = (int)(((long)units * (blockIdx.x + 1)) / gridDim.x);
    const int ntiles_cta = (u1 - u0 + 1) / 2;
    int my_tiles = ntiles_cta > warp ? (ntiles_cta - warp + WARPS - 1) / WARPS : 0;
    // When the CTA has fewer tiles than warps (narrow matrices), the idle warps' ring slots are lent to the working
    // ones: a warp that is alone with a long row range needs more bytes in flight to stream at full speed.
    int mult = 1;
    // Narrow matrices, MH == 1: K relay.  A CTA with at most WARPS/2 tiles gives each tile KS warps; warp (tile, ks)
    // streams steps ks, ks + KS, ... of the tile and computes their products t = (float)D * xs, and the fp32
    // accumulators travel from the warp of step q to the warp of step q + 1 through a mailbox in shared memory, so
    // that every accumulator still sees its groups in ascending order (the bits do not change) while KS rings of
    // copies are in flight per tile instead of one.
    int KS = 1;
    if (MH == 1 && RELAY) while (KS < WARPS && ntiles_cta * KS * 2 <= WARPS) KS *= 2;
    if (KS == 1) while (mult < 4 && ntiles_cta * mult * 2 <= WARPS) mult *= 2;
    const int rtile = warp / KS, rks = warp % KS;            // relay: tile of this warp inside the CTA, first step
    const int depth = STAGES * mult;
    if (KS > 1) my_tiles = (rtile < ntiles_cta && rks < nsteps) ? 1 : 0;
    unsigned char *ring = ring0 + (size_t)warp * mult * STAGES * STEP_BYTES;   // only warps < ntiles_cta use theirs when mult > 1
    const uint32_t ring_u32 = (uint32_t)__cvta_generic_to_shared(ring);
    const size_t wpitch = (size_t)(IN / 2);

    // Producer side of the warp's ring: copies of the next step (tile it, step iq) into slot isl.  One weight-copy
    // instruction covers 32/GS rows x GS*16 contiguous bytes each.
    int it = 0, iq = KS > 1 ? rks : 0, isl = 0;
    auto issue = [&]() {
        if (it < my_tiles) {
            const int base = (u0 + 2 * (KS > 1 ? rtile : warp + it * WARPS)) * 8;
            const uint32_t slot = ring_u32 + (uint32_t)isl * STEP_BYTES;
            constexpr int RPI = 32 / GS;                         // rows per copy instruction
            const int lr = lane / GS, lj = lane % GS;
#pragma unroll
            for (int i = 0; i < 16 / RPI; i++) {
                const int r = i * RPI + lr;
                int row = base + r;
                row = row < OUT ? row : OUT - 1;                 // rows past the end re-read the last row; never stored
                cp_async16_cg(slot + r * (GS * 16) + ((lj ^ swz(r, GS)) << 4), Wq + (size_t)row * wpitch + (size_t)(iq * GS + lj) * 16);
            }
            constexpr int SP = sizeof(ST) == 4 ? GS / 4 : GS / 8;   // 16-byte scale pieces per row
#pragma unroll
            for (int i = 0; i < (16 * SP + 31) / 32; i++) {
                const int pc = i * 32 + lane;
                if (pc < 16 * SP) {
                    const int r = pc / SP, k = pc % SP;
                    int row = base + r;
                    row = row < OUT ? row : OUT - 1;
                    cp_async16_ca(slot + STEP_W + r * (GS * (int)sizeof(ST)) + k * 16,
                                  reinterpret_cast<const unsigned char *>(sw + (size_t)row * nb + iq * GS) + k * 16);
                }
            }
        }
        cp_async_commit();                                        // one group per step, also when empty
        iq += KS;
        if (iq >= nsteps) { iq = KS > 1 ? rks : 0; it++; }
        if (++isl == depth) isl = 0;
    };

    pdl_launch_dependents();
#pragma unroll 1
    for (int s = 0; s < depth - 1; s++) issue();                  // weights only: allowed before the dependency wait
    pdl_wait();

    // ---- stage the activations once per CTA -----------------------------------------------------------------
    // (only rows m < S are read; the rest of the 8*MH rows is zero.)  Two chunks per 128-bit load when xq is 16-byte
    // aligned, else the reference's 4-byte loads.
    // Loads go out in batches (one piece of up to eight rows) before any of them is stored: the compiler cannot tell that the stores to shared
    // memory do not alias the loads, so in a plain loop every load would wait for the store before it (with 8 rows
    // of 5120 elements that serial chain was a quarter of the kernel's time).
    const bool x16 = (reinterpret_cast<uintptr_t>(xq) & 15) == 0;
    constexpr int NT = WARPS * 32, UB = 8;
    if (x16) {
        const int n16 = IN / 16;                                           // 16-byte piece c2 = chunks 2*c2, 2*c2+1
        for (int c2 = tid; c2 < n16; c2 += NT) {
            for (int m0 = 0; m0 < S; m0 += UB) {                           // the same piece of up to UB rows at once
                uint4 v[UB];
#pragma unroll
                for (int u = 0; u < UB; u++)
                    if (m0 + u < S) v[u] = reinterpret_cast<const uint4 *>(xq + (size_t)(m0 + u) * IN)[c2];
#pragma unroll
                for (int u = 0; u < UB; u++) {
                    if (m0 + u < S) {
                        uint32_t e0, o0, e1, o1;
                        split_even_odd(v[u].x, v[u].y, e0, o0);
                        split_even_odd(v[u].z, v[u].w, e1, o1);
                        *reinterpret_cast<uint4 *>(xqp + (size_t)(m0 + u) * pitch2 + 2 * c2) = make_uint4(e0, o0, e1, o1);
                    }
                }
            }
        }
    } else {
        const int n8 = IN / 8;                                             // 8-element chunk c = 4*b + t
        for (int c = tid; c < n8; c += NT) {
            for (int m0 = 0; m0 < S; m0 += UB) {
                uint2 v[UB];
#pragma unroll
                for (int u = 0; u < UB; u++) {
                    if (m0 + u < S) {
                        const uint32_t *src = reinterpret_cast<const uint32_t *>(xq + (size_t)(m0 + u) * IN);
                        v[u] = make_uint2(src[2 * c], src[2 * c + 1]);
                    }
                }
#pragma unroll
                for (int u = 0; u < UB; u++) {
                    if (m0 + u < S) {
                        uint32_t e, od;
                        split_even_odd(v[u].x, v[u].y, e, od);
                        xqp[(size_t)(m0 + u) * pitch2 + c] = make_uint2(e, od);
                    }
                }
            }
        }
    }
    __shared__ float4 relay_box[WARPS / 2][32];
    __shared__ unsigned int relay_flag[WARPS / 2];
    if (tid < WARPS / 2) relay_flag[tid] = 0u;
    for (int i0 = tid; i0 < nb * 8 * MH; i0 += NT * 4) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * NT, b = i / (8 * MH), m = i % (8 * MH);
            v[u] = (i < nb * 8 * MH && m < S) ? xs[(size_t)m * nb + b] : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
            const int i = i0 + u * NT;
            if (i < nb * 8 * MH) sxs[i] = v[u] * 0.0625f;               // exact 1/16: undoes the 16x of the expansion
        }
    }
    __syncthreads();

    float acc[MH][4];
    // ldmatrix row address of this lane inside a slot: matrix i = lane/8 -> rows (i&1)*8.., group 2*jj + (i>>1)
    const int lrow = (lane & 7) + ((lane >> 3) & 1) * 8, lgrp = lane >> 4;
    int csl = 0;
    if (MH == 1 && RELAY && KS > 1) {
        if (my_tiles > 0) {
            volatile unsigned int *flag = &relay_flag[rtile];
            bool alive = true;
            for (int q = rks; q < nsteps && alive; q += KS) {
                issue();
                cp_async_wait<STAGES - 1>();
                __syncwarp();
                const uint32_t slot = ring_u32 + (uint32_t)csl * STEP_BYTES;
                const unsigned char *slot_p = ring + (size_t)csl * STEP_BYTES;
                // ---- all products of this step first: tb[j][i] = (float)D * xs for group j of the step
                float tb[GS][4];
#pragma unroll
                for (int j2 = 0; j2 < GS / 2; j2++) {
                    uint32_t w[4];
                    ldmatrix_x4(slot + lrow * (GS * 16) + (((2 * j2 + lgrp) ^ swz(lrow, GS)) << 4), w[0], w[1], w[2], w[3]);
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        const int j = 2 * j2 + k, b = q * GS + j;
                        uint32_t a0, a1, a2, a3;
                        unpack8_x16(w[2 * k], a0, a2);
                        unpack8_x16(w[2 * k + 1], a1, a3);
                        const uint2 bx = (g < S) ? xqp[(size_t)g * pitch2 + 4 * b + t] : make_uint2(0u, 0u);
                        int c[4];
                        mma_s8(c, a0, a1, a2, a3, bx.x, bx.y);
                        const float2 xv = *reinterpret_cast<const float2 *>(sxs + (size_t)b * 8 + 2 * t);
                        tb[j][0] = (float)c[0] * xv.x; tb[j][1] = (float)c[1] * xv.y;
                        tb[j][2] = (float)c[2] * xv.x; tb[j][3] = (float)c[3] * xv.y;
                    }
                }
                // ---- take the accumulators over from the warp of step q - 1 (bounded wait)
                float a[4] = {0.f, 0.f, 0.f, 0.f};
                if (q > 0) {
                    unsigned int n = 0;
                    while (*flag < (unsigned)q) {
                        if (++n > (1u << 24)) { dev_set_error(0x300u | (unsigned)warp); alive = false; break; }
                    }
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                    __threadfence_block();
                    const float4 v = relay_box[rtile][lane];
                    a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
                }
                // ---- this step's groups, ascending
#pragma unroll
                for (int j4 = 0; j4 < GS / 4; j4++) {
                    float swA[4], swB[4];
                    if (sizeof(ST) == 4) {
                        const float4 fa = *reinterpret_cast<const float4 *>(slot_p + STEP_W + g * (GS * 4) + j4 * 16);
                        const float4 fb = *reinterpret_cast<const float4 *>(slot_p + STEP_W + (g + 8) * (GS * 4) + j4 * 16);
                        swA[0] = fa.x; swA[1] = fa.y; swA[2] = fa.z; swA[3] = fa.w;
                        swB[0] = fb.x; swB[1] = fb.y; swB[2] = fb.z; swB[3] = fb.w;
                    } else {
                        const __half *ha = reinterpret_cast<const __half *>(slot_p + STEP_W + g * (GS * 2) + j4 * 8);
                        const __half *hb = reinterpret_cast<const __half *>(slot_p + STEP_W + (g + 8) * (GS * 2) + j4 * 8);
#pragma unroll
                        for (int j = 0; j < 4; j++) { swA[j] = __half2float(ha[j]); swB[j] = __half2float(hb[j]); }
                    }
#pragma unroll
                    for (int js = 0; js < 4; js++) {
                        const int j = 4 * j4 + js;
                        a[0] = fmaf(tb[j][0], swA[js], a[0]);
                        a[1] = fmaf(tb[j][1], swA[js], a[1]);
                        a[2] = fmaf(tb[j][2], swB[js], a[2]);
                        a[3] = fmaf(tb[j][3], swB[js], a[3]);
                    }
                }
                if (q + 1 < nsteps) {                          // hand over to the warp of step q + 1
                    relay_box[rtile][lane] = make_float4(a[0], a[1], a[2], a[3]);
                    __threadfence_block();
                    __syncwarp();
                    if (lane == 0) *flag = (unsigned)(q + 1);
                } else {                                       // last step: these are the outputs
                    const int base = (u0 + 2 * rtile) * 8;
                    const int lim = min(OUT, u1 * 8);
                    const int m0 = 2 * t, rA = base + g, rB = base + 8 + g;
                    if (rA < lim) {
                        if (m0 < S) store_out<PEER>(Y, oa, OUT, m0, rA, a[0]);
                        if (m0 + 1 < S) store_out<PEER>(Y, oa, OUT, m0 + 1, rA, a[1]);
                    }
                    if (rB < lim) {
                        if (m0 < S) store_out<PEER>(Y, oa, OUT, m0, rB, a[2]);
                        if (m0 + 1 < S) store_out<PEER>(Y, oa, OUT, m0 + 1, rB, a[3]);
                    }
                }
                __syncwarp();                                  // the slot is refilled by the next iteration's copies
                if (++csl == depth) csl = 0;
            }
        }
        my_tiles = 0;                                          // nothing left for the ordinary loop
    }
    for (int ti = 0; ti < my_tiles; ti++) {
#pragma unroll
        for (int h = 0; h < MH; h++) acc[h][0] = acc[h][1] = acc[h][2] = acc[h][3] = 0.f;
        for (int q = 0; q < nsteps; q++) {
            issue();
            if (mult == 1) cp_async_wait<STAGES - 1>();
            else if (mult == 2) cp_async_wait<2 * STAGES - 1>();
            else cp_async_wait<4 * STAGES - 1>();
            __syncwarp();
            const uint32_t slot = ring_u32 + (uint32_t)csl * STEP_BYTES;
            const unsigned char *slot_p = ring + (size_t)csl * STEP_BYTES;
#pragma unroll
            for (int j4 = 0; j4 < GS / 4; j4++) {
                float swA[4], swB[4];
                if (sizeof(ST) == 4) {
                    const float4 a = *reinterpret_cast<const float4 *>(slot_p + STEP_W + g * (GS * 4) + j4 * 16);
                    const float4 b = *reinterpret_cast<const float4 *>(slot_p + STEP_W + (g + 8) * (GS * 4) + j4 * 16);
                    swA[0] = a.x; swA[1] = a.y; swA[2] = a.z; swA[3] = a.w;
                    swB[0] = b.x; swB[1] = b.y; swB[2] = b.z; swB[3] = b.w;
                } else {
                    const __half *a = reinterpret_cast<const __half *>(slot_p + STEP_W + g * (GS * 2) + j4 * 8);
                    const __half *b = reinterpret_cast<const __half *>(slot_p + STEP_W + (g + 8) * (GS * 2) + j4 * 8);
#pragma unroll
                    for (int j = 0; j < 4; j++) { swA[j] = __half2float(a[j]); swB[j] = __half2float(b[j]); }
                }
#pragma unroll
                for (int jj = 0; jj < 2; jj++) {
                    uint32_t w[4];   // rows g (A) / g+8 (B) of groups j0, j0+1: wA0, wB0, wA1, wB1
                    const int j0 = 4 * j4 + 2 * jj;
                    ldmatrix_x4(slot + lrow * (GS * 16) + (((j0 + lgrp) ^ swz(lrow, GS)) << 4), w[0], w[1], w[2], w[3]);
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        const int js = 2 * jj + k, b = q * GS + j0 + k;
                        uint32_t a0, a1, a2, a3;
                        unpack8_x16(w[2 * k], a0, a2);        // rows g   : even -> k-slots 4t.., odd -> k-slots 16+4t..
                        unpack8_x16(w[2 * k + 1], a1, a3);    // rows g+8
#pragma unroll
                        for (int h = 0; h < MH; h++) {
                            // activation row m = 8h + g of this lane; rows beyond S contribute zeros and are not staged
                            const uint2 bx = (8 * h + g < S) ? xqp[(size_t)(8 * h + g) * pitch2 + 4 * b + t] : make_uint2(0u, 0u);
                            int c[4];
                            mma_s8(c, a0, a1, a2, a3, bx.x, bx.y);
                            const float2 xv = *reinterpret_cast<const float2 *>(sxs + (size_t)b * 8 * MH + 8 * h + 2 * t);
                            const float t0 = (float)c[0] * xv.x, t1 = (float)c[1] * xv.y, t2 = (float)c[2] * xv.x, t3 = (float)c[3] * xv.y;
                            acc[h][0] = fmaf(t0, swA[js], acc[h][0]);
                            acc[h][1] = fmaf(t1, swA[js], acc[h][1]);
                            acc[h][2] = fmaf(t2, swB[js], acc[h][2]);
                            acc[h][3] = fmaf(t3, swB[js], acc[h][3]);
                        }
                    }
                }
            }
            __syncwarp();                                  // the slot is refilled by the next iteration's copies
            if (++csl == depth) csl = 0;
        }
        const int base = (u0 + 2 * (warp + ti * WARPS)) * 8;
        const int lim = min(OUT, u1 * 8);
#pragma unroll
        for (int h = 0; h < MH; h++) {
            const int m0 = 8 * h + 2 * t, rA = base + g, rB = base + 8 + g;
            if (rA < lim) {
                if (m0 < S) store_out<PEER>(Y, oa, OUT, m0, rA, acc[h][0]);
                if (m0 + 1 < S) store_out<PEER>(Y, oa, OUT, m0 + 1, rA, acc[h][1]);
            }
            if (rB < lim) {
                if (m0 < S) store_out<PEER>(Y, oa, OUT, m0, rB, acc[h][2]);
                if (m0 + 1 < S) store_out<PEER>(Y, oa, OUT, m0 + 1, rB, acc[h][3]);
            }
        }
    }
    cp_async_wait<0>();
    publish_out<PEER>(oa, 2 * t < S || MH == 2);          // lanes whose columns m = 8h + 2t (+1) exist
}

// Launch plan: groups per step (the largest of 16, 8 that divides the group count), ring depth and rows per pass
// such that the shared-memory plan fits.  Preconditions: K % 256 == 0 (whole steps; 16-byte aligned scale pieces for
// fp32 and fp16), Wq and sw 16-byte aligned, xq 4-byte aligned.
struct Plan { int MH, GS, STAGES; };
constexpr size_t SMEM_LIMIT = 224 * 1024;
inline int env_int(const char *name, int dflt) { const char *e = getenv(name); return e ? atoi(e) : dflt; }
inline bool plan_for(const void *Wq, const void *sw, int IN, int S, Plan *p) {
    const int nb = IN / QBLK;
    if (IN <= 0 || nb % 8 != 0) return false;
    if (!aligned(Wq, 16) || !aligned(sw, 16)) return false;
    static const int want_gs = env_int("W4A8_GEMV_GS", 16);
    static const int want_st = env_int("W4A8_GEMV_STAGES", 0);
    const int MH = S > 8 ? 2 : 1;
    const int gs_opts[2] = {16, 8};
    for (int gi = 0; gi < 2; gi++) {
        const int GS = gs_opts[gi];
        if (GS > want_gs || nb % GS != 0) continue;
        const int st_opts[3] = {GS == 16 ? 4 : 8, GS == 16 ? 3 : 6, GS == 16 ? 2 : 3};
        for (int si = 0; si < 3; si++)
            if (st_opts[si] <= (want_st > 0 ? want_st : (GS == 16 ? 2 : 3)))
            if (smem_bytes(MH, S, nb, GS, st_opts[si]) <= SMEM_LIMIT) { p->MH = MH; p->GS = GS; p->STAGES = st_opts[si]; return true; }
    }
    return false;
}

template <int MH, int GS, int STAGES, typename ST, bool PEER>
inline int launch_p(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int IN, int OUT, int S,
                    cudaStream_t st, const OutArgs &oa) {
    const int nb = IN / QBLK;
    const size_t smem = smem_bytes(MH, S, nb, GS, STAGES);
    auto kern = gemv_w4a8_mma_kernel<MH, GS, STAGES, ST, PEER>;
    static PerDevice<size_t> configured_dev;            // grow-only; the opt-in is a per-device function attribute
    size_t &configured = configured_dev.get();
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "gemv_mma smem opt-in");
        configured = smem;
    }
    const int units = (OUT + 7) / 8;
    long want = (units + 1) / 2;                         // at least one 16-row tile per CTA
    long cap = sm_count();                               // one persistent CTA per SM
    const dim3 grid((unsigned)(want < cap ? want : cap));
    cudaError_t le = launch_pdl(kern, grid, dim3(WARPS * 32), smem, st, xq, xs, Wq, sw, Y, IN, OUT, S, oa);
    if (le != cudaSuccess) return cuda_fail(le, "gemv_w4a8_mma launch");
    return launch_status("gemv_w4a8_mma");
}

template <int MH, int GS, int STAGES, typename ST>
inline int launch_t(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int IN, int OUT, int S,
                    cudaStream_t st, const OutArgs &oa) {
    if (oa.peers) return launch_p<MH, GS, STAGES, ST, true>(xq, xs, Wq, sw, Y, IN, OUT, S, st, oa);
    return launch_p<MH, GS, STAGES, ST, false>(xq, xs, Wq, sw, Y, IN, OUT, S, st, oa);
}

template <typename ST>
inline int launch_st(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int IN, int OUT, int S,
                     const Plan &p, cudaStream_t st, const OutArgs &oa) {
#define W4A8_MMA_CASE(MH_, GS_, ST_) \
    if (p.MH == MH_ && p.GS == GS_ && p.STAGES == ST_) return launch_t<MH_, GS_, ST_, ST>(xq, xs, Wq, sw, Y, IN, OUT, S, st, oa);
    W4A8_MMA_CASE(1, 16, 4) W4A8_MMA_CASE(1, 16, 3) W4A8_MMA_CASE(1, 16, 2) W4A8_MMA_CASE(1, 8, 8) W4A8_MMA_CASE(1, 8, 6) W4A8_MMA_CASE(1, 8, 3)
    W4A8_MMA_CASE(2, 16, 4) W4A8_MMA_CASE(2, 16, 3) W4A8_MMA_CASE(2, 16, 2) W4A8_MMA_CASE(2, 8, 8) W4A8_MMA_CASE(2, 8, 6) W4A8_MMA_CASE(2, 8, 3)
#undef W4A8_MMA_CASE
    return fail(W4A8_ERR_UNSUPPORTED, "gemv_mma: no kernel for plan MH=%d GS=%d STAGES=%d", p.MH, p.GS, p.STAGES);
}

inline int launch(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int IN, int OUT, int S,
                  int scale_dtype, const Plan &p, cudaStream_t st, const OutArgs &oa = OutArgs()) {
    if (scale_dtype == 1) return launch_st<__half>(xq, xs, Wq, (const __half *)sw, Y, IN, OUT, S, p, st, oa);
    return launch_st<float>(xq, xs, Wq, (const float *)sw, Y, IN, OUT, S, p, st, oa);
}

}  // namespace gemv_mma
}  // namespace w4a8
