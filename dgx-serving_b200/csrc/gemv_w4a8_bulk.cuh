// W4A8 decode GEMV for ONE activation row, weights streamed by bulk asynchronous copies (cp.async.bulk) into a
// shared-memory ring.  Same product and the same fp32 order as the dp4a kernel of csrc/gemv_w4a8.cuh (the
// reference's kernels/gemv_w4a8.cuh:119-151): lane l of the warp that owns a row takes groups l, l+32, ... in
// ascending order, acc = fma((xs*sw)/16, (float)(16*D), acc), then the shfl_down tree — bit-identical results.
//
// Why a second M=1 kernel: a 10-microsecond stream is bound by the bytes it keeps in flight and by what a launch
// costs before and after its steady state.  With register loads a lane holds five 16-byte loads, 24 warps per SM ->
// about 60 KB per SM, and every byte in flight holds a register and an issue slot.  Here the rows of a CTA are
// contiguous in memory, so ROWS consecutive weight rows are one contiguous block: one elected thread issues one bulk
// copy per block (plus one for the block's scales) and the copy engine keeps the whole ring (4 stages of 12 rows,
// about 150 KB per SM) in flight.  The activation row lives in registers (a lane always meets the same groups), so
// the consumers read only weights and scales from shared memory.  Measured on K=5120, N=17408: 10.2 us against
// 11.5 us for the register-load kernel; K=5120, N=151936: 71 us = 6.9 TB/s.  One CTA per SM with 12 consumer warps
// measured best; two smaller CTAs per SM, or rings deeper than 4 stages, were slower.
//
// Preconditions (else the caller uses another kernel): S = 1, K % 128 = 0 (K % 256 = 0 with fp16 scales: scale rows
// are multiples of 16 bytes), K <= 8192, Wq and sw 16-byte aligned.  No expert grouping.
#pragma once
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "peer_allgather.cuh"

namespace w4a8 {
namespace gemv_bulk {

#ifndef W4A8_BULK_CW
#define W4A8_BULK_CW 12
#endif
constexpr int CW = W4A8_BULK_CW;        // consumer warps per CTA
#ifndef W4A8_BULK_RPW
#define W4A8_BULK_RPW 1
#endif
constexpr int RPW = W4A8_BULK_RPW;      // rows per warp and stage, processed interleaved (independent chains)
constexpr int ROWS = CW * RPW;          // weight rows per ring stage
constexpr int MAX_STAGES = 8;
constexpr int BAR_BYTES = 256;          // full[MAX_STAGES], empty[MAX_STAGES], padding
// Consumer warps come in G groups of CW; group g takes the ring stages g, g + G, ...  A consumer warp needs about two
// thousand cycles per row (shared-memory loads, the dp4a chain, the barrier hand-offs), longer than the copies need to
// deliver a stage, so one group alone leaves HBM waiting for the consumers; two groups work on two stages at once.
// The ring depth is a multiple of G, so a ring slot is always used by the same group, use after use (a parity wait
// on an mbarrier may never be more than one phase ahead).
#ifndef W4A8_BULK_GROUPS
#define W4A8_BULK_GROUPS 2
#endif
constexpr int MAX_G = W4A8_BULK_GROUPS;
constexpr int THREADS = (MAX_G * CW + 1) * 32;

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

struct Ring {
    int stage = 0, depth;
    uint32_t phase = 0;
    __device__ explicit Ring(int d) : depth(d) {}
    __device__ void advance() { if (++stage == depth) { stage = 0; phase ^= 1u; } }
};

// Up to MAX_MATS matrices that share one activation row (gate + up, q + k + v): one launch, the CTAs of the grid
// are divided between the matrices in proportion to their rows (cta0[i] = first CTA of matrix i).
constexpr int MAX_MATS = 4;
struct Mats {
    const uint8_t *Wq[MAX_MATS];
    const void *sw[MAX_MATS];
    float *Y[MAX_MATS];
    int OUT[MAX_MATS];
    int cta0[MAX_MATS + 1];
    int count;
};

// NG = groups per lane = ceil(K / 1024).
// PEER: outputs go to every rank's arena and the last CTA publishes the step's epoch (peer_allgather.cuh); single matrix.
template <int NG, typename ST, bool PEER>
__global__ void __launch_bounds__(THREADS) gemv_w4a8_bulk_kernel(
    const int8_t *__restrict__ xq, const float *__restrict__ xs, const Mats mats, int IN, int nstages, int G, OutArgs oa) {
    int mi = 0;
    while (mi + 1 < mats.count && (int)blockIdx.x >= mats.cta0[mi + 1]) mi++;
    const uint8_t *__restrict__ Wq = mats.Wq[mi];
    const ST *__restrict__ sw = static_cast<const ST *>(mats.sw[mi]);
    float *__restrict__ Y = mats.Y[mi];
    const int OUT = mats.OUT[mi];
    const int cta = (int)blockIdx.x - mats.cta0[mi], nctas = mats.cta0[mi + 1] - mats.cta0[mi];
    extern __shared__ __align__(128) unsigned char smem[];
    const int nb = IN / QBLK;
    const uint32_t wrow = (uint32_t)IN / 2, srow = (uint32_t)nb * sizeof(ST);
    const uint32_t stage_bytes = ROWS * (wrow + srow);
    const uint32_t smem_u32 = ptx::smem_u32(smem);
    auto FULL = [&](int i) { return smem_u32 + 8u * i; };
    auto EMPTY = [&](int i) { return smem_u32 + 8u * (MAX_STAGES + i); };
    unsigned char *ring = smem + BAR_BYTES;
    const uint32_t ring_u32 = smem_u32 + BAR_BYTES;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // rows [r0, r1) of this CTA: a balanced contiguous partition of OUT over the grid
    const int r0 = (int)(((long)OUT * cta) / nctas), r1 = (int)(((long)OUT * (cta + 1)) / nctas);
    const int nchunks = (r1 - r0 + ROWS - 1) / ROWS;

    if (tid == 0) {
        for (int i = 0; i < nstages; i++) { ptx::mbar_init(FULL(i), 1); ptx::mbar_init(EMPTY(i), CW); }
        ptx::mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == G * CW) {
        // ---------------- producer: one thread, weights and scales only (no dependency on the previous kernel) ----
        if (lane == 0) {
            Ring r(nstages);
            bool ok = true;
            for (int c = 0; c < nchunks; c++) {
                if (!ptx::mbar_wait(EMPTY(r.stage), r.phase ^ 1u)) { dev_set_error(0x400u | 1u); ok = false; break; }
                const int row = r0 + c * ROWS;
                const uint32_t rows = (uint32_t)min(ROWS, r1 - row);
                const uint32_t dst = ring_u32 + (uint32_t)r.stage * stage_bytes;
                ptx::mbar_arrive_expect_tx(FULL(r.stage), rows * (wrow + srow));
                bulk_g2s(dst, Wq + (size_t)row * wrow, rows * wrow, FULL(r.stage));
                bulk_g2s(dst + ROWS * wrow, reinterpret_cast<const unsigned char *>(sw) + (size_t)row * srow, rows * srow, FULL(r.stage));
                r.advance();
            }
            if (!ok) {  // give copies already in flight time to land before the CTA's shared memory goes away
                const long long t0 = clock64();
                while (clock64() - t0 < (1ll << 21)) { }
            }
        }
    } else {
        // ---------------- consumers: warp w owns row w of every stage --------------------------------------------
        pdl_wait();   // the activations come from the kernel before this one
        const bool x16 = (reinterpret_cast<uintptr_t>(xq) & 15) == 0;
        uint32_t xe[NG][4], xo[NG][4];
        float xsr[NG];
#pragma unroll
        for (int j = 0; j < NG; j++) {
            const int b = lane + 32 * j;
            uint32_t v[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
            xsr[j] = 0.f;
            if (b < nb) {
                if (x16) {
                    const uint4 *src = reinterpret_cast<const uint4 *>(xq + (size_t)b * QBLK);
                    const uint4 a = src[0], c4 = src[1];
                    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c4.x; v[5] = c4.y; v[6] = c4.z; v[7] = c4.w;
                } else {
                    const uint32_t *src = reinterpret_cast<const uint32_t *>(xq + (size_t)b * QBLK);
#pragma unroll
                    for (int i = 0; i < 8; i++) v[i] = src[i];
                }
                xsr[j] = xs[b];
            }
#pragma unroll
            for (int i = 0; i < 4; i++) split_even_odd(v[2 * i], v[2 * i + 1], xe[j][i], xo[j][i]);
        }
        const int grp = warp / CW, lw = warp - grp * CW;        // group and warp inside the group
        for (int c = grp; c < nchunks; c += G) {
            Ring r(nstages);
            r.stage = c % nstages; r.phase = (uint32_t)(c / nstages) & 1u;
            if (!ptx::mbar_wait_warp(FULL(r.stage), r.phase)) { dev_set_error(0x400u | 2u); break; }
            const int row = r0 + c * ROWS + lw;                // this warp's rows: row + CW * i
            if (row < r1) {
                const unsigned char *stage_p = ring + (size_t)r.stage * stage_bytes;
                float acc[RPW];
#pragma unroll
                for (int i = 0; i < RPW; i++) acc[i] = 0.f;
#pragma unroll
                for (int j = 0; j < NG; j++) {
                    const int b = lane + 32 * j;
                    if (b < nb) {
#pragma unroll
                        for (int i = 0; i < RPW; i++) {
                            const int lr = lw + CW * i;            // row inside the stage (rows past r1 hold stale bytes: never stored)
                            const uint4 wv = *reinterpret_cast<const uint4 *>(stage_p + (size_t)lr * wrow + (size_t)b * 16);
                            const float s = sval(reinterpret_cast<const ST *>(stage_p + (size_t)ROWS * wrow + (size_t)lr * srow)[b]);
                            uint32_t e0, o0, e1, o1, e2, o2, e3, o3;
                            unpack8_x16(wv.x, e0, o0); unpack8_x16(wv.y, e1, o1);
                            unpack8_x16(wv.z, e2, o2); unpack8_x16(wv.w, e3, o3);
                            int d = __dp4a((int)xe[j][0], (int)e0, 0);
                            d = __dp4a((int)xo[j][0], (int)o0, d);
                            d = __dp4a((int)xe[j][1], (int)e1, d);
                            d = __dp4a((int)xo[j][1], (int)o1, d);
                            d = __dp4a((int)xe[j][2], (int)e2, d);
                            d = __dp4a((int)xo[j][2], (int)o2, d);
                            d = __dp4a((int)xe[j][3], (int)e3, d);
                            d = __dp4a((int)xo[j][3], (int)o3, d);      // d = 16 * D[o,b], exact
                            const float sc = (xsr[j] * s) * 0.0625f;    // exact 1/16
                            acc[i] = fmaf(sc, (float)d, acc[i]);
                        }
                    }
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1)
#pragma unroll
                    for (int i = 0; i < RPW; i++) acc[i] += __shfl_down_sync(0xffffffffu, acc[i], off);
                if (lane == 0) {
#pragma unroll
                    for (int i = 0; i < RPW; i++)
                        if (row + CW * i < r1) store_out<PEER>(Y, oa, OUT, 0, row + CW * i, acc[i]);
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(EMPTY(r.stage));
        }
    }
    publish_out<PEER>(oa, lane == 0 && warp < G * CW);
}

struct Plan { int NG, stages, ctas_per_sm, groups; size_t smem; };

// Ring depth and residency for a row of IN elements, or false when the shape is not served here.
inline bool plan_for(const void *xq, const void *Wq, const void *sw, int IN, int scale_dtype, Plan *p) {
    const int nb = IN / QBLK;
    const int need = scale_dtype == 1 ? 256 : 128;
    if (IN <= 0 || IN % need != 0 || nb > 256) return false;
    if (!aligned(Wq, 16) || !aligned(sw, 16) || !aligned(xq, 4)) return false;
    const size_t stage = (size_t)ROWS * ((size_t)IN / 2 + (size_t)nb * (scale_dtype == 1 ? 2 : 4));
    static const int want_st = [] { const char *e = getenv("W4A8_GEMV_BULK_STAGES"); return e ? atoi(e) : 0; }();
    static const int want_occ = [] { const char *e = getenv("W4A8_GEMV_BULK_OCC"); return e ? atoi(e) : 1; }();
    int occ = want_occ >= 2 ? 2 : 1;
    int st = (int)((112u * 1024u - BAR_BYTES) / stage);
    if (occ == 2 && st < 2) occ = 1;
    if (occ == 1) st = (int)((224u * 1024u - BAR_BYTES) / stage);
    if (st > (occ == 1 ? 4 : MAX_STAGES)) st = occ == 1 ? 4 : MAX_STAGES;   // one CTA per SM: deeper than 4 stages measured slower
    if (want_st > 0 && want_st < st) st = want_st;
    if (st < 2) return false;
    static const int want_g = [] { const char *e = getenv("W4A8_GEMV_BULK_GROUPS"); return e ? atoi(e) : MAX_G; }();
    int g = want_g < 1 ? 1 : (want_g > MAX_G ? MAX_G : want_g);
    if (occ == 2) g = 1;
    while (g > 1 && st % g != 0) st--;                      // ring depth: a multiple of the group count
    if (st < g) g = 1;
    p->NG = (nb + 31) / 32; p->stages = st; p->ctas_per_sm = occ; p->groups = g; p->smem = BAR_BYTES + (size_t)st * stage;
    return true;
}

template <int NG, typename ST, bool PEER>
inline int launch_p(const int8_t *xq, const float *xs, const Mats &mats_in, int IN, const Plan &p, cudaStream_t st, const OutArgs &oa) {
    auto kern = gemv_w4a8_bulk_kernel<NG, ST, PEER>;
    static PerDevice<size_t> configured_dev;            // grow-only; the opt-in is a per-device function attribute
    size_t &configured = configured_dev.get();
    if (p.smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem);
        if (e != cudaSuccess) return cuda_fail(e, "gemv_bulk smem opt-in");
        configured = p.smem;
    }
    // grid: one persistent CTA per SM (p.ctas_per_sm of them), fewer when there are not enough rows; the CTAs are
    // dealt to the matrices in proportion to their rows, at least one each
    Mats m = mats_in;
    long total = 0;
    for (int i = 0; i < m.count; i++) total += m.OUT[i];
    const long want = (total + ROWS - 1) / ROWS, cap = (long)sm_count() * p.ctas_per_sm;
    long grid = want < cap ? want : cap;
    if (grid < m.count) grid = m.count;
    m.cta0[0] = 0;
    long acc_rows = 0;
    for (int i = 0; i < m.count; i++) {
        acc_rows += m.OUT[i];
        long end = (grid * acc_rows + total / 2) / total;
        if (end < m.cta0[i] + 1) end = m.cta0[i] + 1;                       // at least one CTA per matrix
        const long room = grid - (m.count - 1 - i);                        // leave one for each matrix still to come
        if (end > room) end = room;
        m.cta0[i + 1] = (int)end;
    }
    m.cta0[m.count] = (int)grid;
    cudaError_t le = launch_pdl(kern, dim3((unsigned)grid), dim3((p.groups * CW + 1) * 32), p.smem, st, xq, xs, m, IN, p.stages, p.groups, oa);
    if (le != cudaSuccess) return cuda_fail(le, "gemv_w4a8_bulk launch");
    return launch_status("gemv_w4a8_bulk");
}

template <int NG, typename ST>
inline int launch_t(const int8_t *xq, const float *xs, const Mats &m, int IN, const Plan &p, cudaStream_t st, const OutArgs &oa) {
    if (oa.peers) return launch_p<NG, ST, true>(xq, xs, m, IN, p, st, oa);
    return launch_p<NG, ST, false>(xq, xs, m, IN, p, st, oa);
}

template <typename ST>
inline int launch_st(const int8_t *xq, const float *xs, const Mats &m, int IN, const Plan &p, cudaStream_t st, const OutArgs &oa) {
    switch (p.NG) {
        case 1: return launch_t<1, ST>(xq, xs, m, IN, p, st, oa);
        case 2: return launch_t<2, ST>(xq, xs, m, IN, p, st, oa);
        case 3: return launch_t<3, ST>(xq, xs, m, IN, p, st, oa);
        case 4: return launch_t<4, ST>(xq, xs, m, IN, p, st, oa);
        case 5: return launch_t<5, ST>(xq, xs, m, IN, p, st, oa);
        case 6: return launch_t<6, ST>(xq, xs, m, IN, p, st, oa);
        case 7: return launch_t<7, ST>(xq, xs, m, IN, p, st, oa);
        case 8: return launch_t<8, ST>(xq, xs, m, IN, p, st, oa);
    }
    return fail(W4A8_ERR_UNSUPPORTED, "gemv_bulk: no kernel for %d groups per lane", p.NG);
}

inline int launch_multi(const int8_t *xq, const float *xs, const Mats &m, int IN, int scale_dtype, const Plan &p, cudaStream_t st,
                        const OutArgs &oa = OutArgs()) {
    if (scale_dtype == 1) return launch_st<__half>(xq, xs, m, IN, p, st, oa);
    return launch_st<float>(xq, xs, m, IN, p, st, oa);
}

inline int launch(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int IN, int OUT,
                  int scale_dtype, const Plan &p, cudaStream_t st, const OutArgs &oa = OutArgs()) {
    Mats m = {};
    m.Wq[0] = Wq; m.sw[0] = sw; m.Y[0] = Y; m.OUT[0] = OUT; m.count = 1;
    return launch_multi(xq, xs, m, IN, scale_dtype, p, st, oa);
}

}  // namespace gemv_bulk
}  // namespace w4a8
