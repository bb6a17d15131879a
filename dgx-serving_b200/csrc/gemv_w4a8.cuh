// W4A8 decode GEMV family for sm_100a: Y[s,o] = sum_b xs[s,b]*sw[o,b] * D[s,o,b],
// D[s,o,b] = sum_{k in group b} xq[s,k] * (Wq[o,k] - 8), the semantics of the reference's
// kernels/gemv_w4a8.cuh:24-49 (plain), :54-110 (mlp), :119-151 (SB), :182-347 (g4) and
// kernels/gemm_batch.cuh:177-231 (batch).  HBM-bound: the packed weights and their scales are read
// exactly once per launch for all S rows.
//
// Work layout.  One quantization group (32 int4 = 16 bytes) is one 128-bit load.  A warp owns one
// output row o; lane l owns groups b = l, l+32, l+64, ... so each warp-wide load covers 512 contiguous
// bytes of the row.  The lane computes the whole 32-element integer dot of its group (8 dp4a per
// activation row), converts it once and scales it with xs[s,b]*sw[o,b].
//
// fp32 evaluation order (fixed, independent of S and of which kernel variant runs):
//   chain c = b mod 32:  acc_c = fma(xs[s,b]*sw[o,b], (float)D[s,o,b], acc_c), b = c, c+32, ... ascending
//   result = tree over the 32 chains exactly as a shfl_down 16,8,4,2,1 reduction leaves it in lane 0.
// (The reference's own GEMV order, tied to its 4-byte-per-lane loads, differs in the last bits; its
// tests compare families with max|d|/rms < 1e-5, tests/test_gemm_mmq.cu:28.)
#pragma once
#include "common.cuh"
#include "fused_quantize.cuh"
#include "peer_allgather.cuh"

namespace w4a8 {

constexpr int GEMV_WARPS = 8;      // warps (= output rows) per CTA
constexpr int SHORT_WARPS = 4;     // warps per CTA of the short-row kernel: at about 78 registers six such CTAs fit an SM, and a
                                   // grouped launch's CTAs-per-slot then fill 94 % of a wave (three 8-warp CTAs: 86 %)
constexpr int GEMV_MT_MAX = 4;     // activation rows handled per pass of the dp4a kernel

// Grouped-expert addressing (idx == nullptr: plain dense GEMV).  Expert e's weights start
// e*(OUT*IN/2) bytes into Wq and its scales e*(OUT*IN/32) elements into sw, the indexing of the
// reference's kernels/moe_fused.cuh:21-24; slot = token*topk + k.
struct GroupedArgs {
    const int32_t *idx = nullptr;
    int topk = 1, x_per_slot = 0, num_experts = 0, nslots = 1;
    int expert_base = 0;   // experts [expert_base, expert_base + num_experts) live in this Wq / sw (an expert shard)
    int shard_world = 1;   // expert shard: about 1 / shard_world of the slots are this rank's, the other slots' CTAs exit at once
    // Short-row kernels only: the slot's activation row is produced in the kernel's prologue instead of being read from
    // xq / xs.  1: quantize_x of row slot / topk of src_f32 [tokens][IN]; 2: activation (act 0 SwiGLU, 1 GeGLU) of row slot
    // of src_f32 [nslots][2 IN] (gate | up), then quantize_x.  The first CTA of every slot also stores the row to
    // xq_out / xs_out (row slot / topk resp. slot), so the stage can still be read back.
    int src_mode = 0, act = 0;
    const float *src_f32 = nullptr;
    int8_t *xq_out = nullptr;
    float *xs_out = nullptr;
};

__device__ __forceinline__ uint4 ldg_w16(const uint8_t *p, bool a16) {
    if (a16) return __ldcs(reinterpret_cast<const uint4 *>(p));  // streamed once: evict-first
    const uint32_t *q = reinterpret_cast<const uint32_t *>(p);
    return make_uint4(q[0], q[1], q[2], q[3]);
}

// MT  activation rows per pass (1..4), U = groups per lane loaded as one batch.
// Persistent CTAs: the grid is sized to the device (a few CTAs per SM) and every CTA owns a contiguous
// range of output rows, so the activations are staged once per CTA, not once per 8 rows.  Warp w of the
// CTA takes rows r0+w, r0+w+8, ...; the (row, batch) items of a warp form one flat sequence that is
// software-pipelined: the 128-bit weight loads and scale loads of item i+1 are issued before item i is
// unpacked and accumulated, so every lane keeps two batches of loads in flight.
// Shared memory: the MT activation rows, re-ordered once per CTA so that every group is two 16-byte
// pieces [e0 o0 e1 o1] and [e2 o2 e3 o3] (ew/ow = even/odd elements of the w-th 8-element chunk), the
// order unpack8_x16 produces for the weights; the pieces live in two planes so that consecutive lanes
// read consecutive 16-byte words (no bank conflicts).  Then xs[MT][nb].
template <int U, typename ST>
struct GemvBatch {
    uint4 w[U];
    float s[U];
};

// Scale of group b of a row.  fp16 scales are fetched as the aligned 32-bit word that holds the pair (b & ~1, b | 1)
// when the row start is 4-byte aligned (two-byte loads cost the same requests for half the bytes).
__device__ __forceinline__ float load_scale(const float *swrow, int b) { return swrow[b]; }
__device__ __forceinline__ float load_scale(const __half *swrow, int b) {
    if ((reinterpret_cast<uintptr_t>(swrow) & 3) == 0) {
        const uint32_t w = reinterpret_cast<const uint32_t *>(swrow)[b >> 1];
        return __half2float(__ushort_as_half((unsigned short)((b & 1) ? (w >> 16) : (w & 0xFFFFu))));
    }
    return __half2float(swrow[b]);
}

template <int U, typename ST>
__device__ __forceinline__ void gemv_load_batch(GemvBatch<U, ST> &bt, const uint8_t *__restrict__ wrow,
                                                const ST *__restrict__ swrow, int slot0, int lane, int nb, bool a16) {
#pragma unroll
    for (int u = 0; u < U; u++) {
        const int b = lane + 32 * (slot0 + u);
        if (b < nb) { bt.w[u] = ldg_w16(wrow + 16 * b, a16); bt.s[u] = load_scale(swrow, b); }
        else { bt.w[u] = make_uint4(0, 0, 0, 0); bt.s[u] = 0.f; }
    }
}

template <int MT, int U, typename ST>
__device__ __forceinline__ void gemv_compute_batch(const GemvBatch<U, ST> &bt, float (&acc)[MT], const uint4 *plane0,
                                                   const uint4 *plane1, const float *sxs, int slot0, int lane, int nb) {
#pragma unroll
    for (int u = 0; u < U; u++) {
        const int b = lane + 32 * (slot0 + u);
        if (b < nb) {
            uint32_t e0, o0, e1, o1, e2, o2, e3, o3;
            unpack8_x16(bt.w[u].x, e0, o0); unpack8_x16(bt.w[u].y, e1, o1);
            unpack8_x16(bt.w[u].z, e2, o2); unpack8_x16(bt.w[u].w, e3, o3);
#pragma unroll
            for (int m = 0; m < MT; m++) {
                const uint4 xa = plane0[m * nb + b], xb = plane1[m * nb + b];
                int d = __dp4a((int)xa.x, (int)e0, 0);
                d = __dp4a((int)xa.y, (int)o0, d);
                d = __dp4a((int)xa.z, (int)e1, d);
                d = __dp4a((int)xa.w, (int)o1, d);
                d = __dp4a((int)xb.x, (int)e2, d);
                d = __dp4a((int)xb.y, (int)o2, d);
                d = __dp4a((int)xb.z, (int)e3, d);
                d = __dp4a((int)xb.w, (int)o3, d);      // d = 16 * D[m,o,b], exact
                const float sc = (sxs[m * nb + b] * bt.s[u]) * 0.0625f;   // exact 1/16
                acc[m] = fmaf(sc, (float)d, acc[m]);
            }
        }
    }
}

template <int MT, int U, typename ST, bool PEER>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_w4a8_dp4a_kernel(
    const int8_t *__restrict__ xq, const float *__restrict__ xs, const uint8_t *__restrict__ Wq,
    const ST *__restrict__ sw, float *__restrict__ Y, int IN, int OUT, int S, bool w_a16, GroupedArgs ga, OutArgs oa) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int nb = IN / QBLK;
    if (ga.idx) {  // grouped experts: blockIdx.y = slot, one activation row against that slot's expert
        const int slot = blockIdx.y;
        pdl_wait();   // the routing indices are written by an earlier kernel of the stream (router / top-k): wait first
        const int e = ga.idx[slot] - ga.expert_base;
        if (e < 0 || e >= ga.num_experts) return;   // invalid id, or another rank's expert: the slot's output row is left untouched
        const int row = ga.x_per_slot ? slot : slot / ga.topk;
        xq += (size_t)row * IN;
        xs += (size_t)row * nb;
        Wq += (size_t)e * ((size_t)OUT * (IN / 2));
        sw += (size_t)e * ((size_t)OUT * nb);
        Y += (size_t)slot * OUT;
    }
    uint4 *plane0 = reinterpret_cast<uint4 *>(smem_raw);            // [MT][nb]
    uint4 *plane1 = plane0 + (size_t)MT * nb;                       // [MT][nb]
    float *sxs = reinterpret_cast<float *>(plane1 + (size_t)MT * nb);  // [MT][nb]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // rows [r0, r1) of this CTA: a balanced contiguous partition of OUT over gridDim.x
    const int r0 = (int)(((long)OUT * blockIdx.x) / gridDim.x), r1 = (int)(((long)OUT * (blockIdx.x + 1)) / gridDim.x);
    const int nbatch = ((nb + 31) / 32 + U - 1) / U;                // batches per row
    const int nrows_w = (r1 - r0 - warp + GEMV_WARPS - 1) / GEMV_WARPS;   // rows of this warp (may be <= 0)
    const int nitems = nrows_w > 0 ? nrows_w * nbatch : 0;
    const size_t wpitch = (size_t)(IN / 2);

    // The first batch of weight loads goes out before the activations are staged.
    GemvBatch<U, ST> ba, bb;
    pdl_launch_dependents();
    if (nitems > 0) gemv_load_batch<U, ST>(ba, Wq + (size_t)(r0 + warp) * wpitch, sw + (size_t)(r0 + warp) * nb, 0, lane, nb, w_a16);
    // Everything above read only the weights and their scales.  The activations (written by the quantize kernel
    // that precedes this launch in the stream) and Y may only be touched once the previous kernel is complete.
    pdl_wait();

    // Stage activations: one task = one 8-element chunk (two 4-byte loads, like the reference's x0/x1).
#pragma unroll
    for (int m = 0; m < MT; m++) {
        // loads in batches of UB ahead of the stores: the compiler cannot tell that the shared-memory stores do not
        // alias the loads, and a long row would otherwise pay one L2 round trip per chunk
        constexpr int NT = GEMV_WARPS * 32, UB = 8;
        for (int c0 = tid; c0 < IN / 8; c0 += NT * UB) {
            uint32_t x0[UB], x1[UB];
#pragma unroll
            for (int u = 0; u < UB; u++) {
                const int c = c0 + u * NT;
                x0[u] = 0; x1[u] = 0;
                if (m < S && c < IN / 8) {
                    const uint32_t *src = reinterpret_cast<const uint32_t *>(xq + (size_t)m * IN + 8 * c);
                    x0[u] = src[0]; x1[u] = src[1];
                }
            }
#pragma unroll
            for (int u = 0; u < UB; u++) {
                const int c = c0 + u * NT;
                if (c < IN / 8) {
                    uint32_t e, od;
                    split_even_odd(x0[u], x1[u], e, od);
                    const int b = c >> 2, w = c & 3;
                    uint2 *dst = reinterpret_cast<uint2 *>((w < 2 ? plane0 : plane1) + (size_t)m * nb + b) + (w & 1);
                    *dst = make_uint2(e, od);
                }
            }
        }
        for (int b0 = tid; b0 < nb; b0 += NT * 4) {
            float v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) { const int b = b0 + u * NT; v[u] = (m < S && b < nb) ? xs[(size_t)m * nb + b] : 0.f; }
#pragma unroll
            for (int u = 0; u < 4; u++) { const int b = b0 + u * NT; if (b < nb) sxs[m * nb + b] = v[u]; }
        }
    }
    __syncthreads();

    float acc[MT];
#pragma unroll
    for (int m = 0; m < MT; m++) acc[m] = 0.f;

    // item i: row = r0 + warp + 8*(i / nbatch), batch = i % nbatch.  Two items per trip so that the two
    // register buffers alternate without copies.
    int row = r0 + warp, batch = 0;
    auto advance = [&](int &r, int &bi) { if (++bi == nbatch) { bi = 0; r += GEMV_WARPS; } };
    auto finish_row = [&](int r) {
#pragma unroll
        for (int m = 0; m < MT; m++) {
            float v = acc[m];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
            if (lane == 0 && m < S) store_out<PEER>(Y, oa, OUT, m, r, v);
            acc[m] = 0.f;
        }
    };
    for (int i = 0; i < nitems; i += 2) {
        int nrow = row, nbt = batch;
        advance(nrow, nbt);
        if (i + 1 < nitems) gemv_load_batch<U, ST>(bb, Wq + (size_t)nrow * wpitch, sw + (size_t)nrow * nb, nbt * U, lane, nb, w_a16);
        gemv_compute_batch<MT, U, ST>(ba, acc, plane0, plane1, sxs, batch * U, lane, nb);
        if (batch == nbatch - 1) finish_row(row);
        if (i + 1 >= nitems) break;
        row = nrow; batch = nbt;
        advance(nrow, nbt);
        if (i + 2 < nitems) gemv_load_batch<U, ST>(ba, Wq + (size_t)nrow * wpitch, sw + (size_t)nrow * nb, nbt * U, lane, nb, w_a16);
        gemv_compute_batch<MT, U, ST>(bb, acc, plane0, plane1, sxs, batch * U, lane, nb);
        if (batch == nbatch - 1) finish_row(row);
        row = nrow; batch = nbt;
    }
    publish_out<PEER>(oa, lane == 0);
}

template <int MT, int U, typename ST, bool PEER>
inline int launch_gemv_dp4a_p(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y,
                              int IN, int OUT, int S, cudaStream_t st, const GroupedArgs &ga, const OutArgs &oa) {
    const int nb = IN / QBLK;
    const size_t smem = (size_t)MT * IN + (size_t)MT * nb * sizeof(float);
    auto kern = gemv_w4a8_dp4a_kernel<MT, U, ST, PEER>;
    if (smem > 48 * 1024) {
        static PerDevice<size_t> configured_dev;        // grow-only; the opt-in is a per-device function attribute
        size_t &configured = configured_dev.get();
        if (smem > configured) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return cuda_fail(e, "gemv smem opt-in");
            configured = smem;
        }
    }
    // Persistent: as many CTAs as are resident at once (fewer when there are not enough rows, or when grouped
    // slots already fill the GPU).  Residency is asked of the runtime once per kernel variant and smem size.
    struct Occ { size_t smem_plus1; int occ; };          // per device: another GPU may answer differently
    static PerDevice<Occ> occ_dev;
    Occ &oc = occ_dev.get();
    size_t occ_smem = oc.smem_plus1 - 1;
    int occ = oc.occ > 0 ? oc.occ : 1;
    if (oc.smem_plus1 == 0 || occ_smem != smem) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, GEMV_WARPS * 32, smem);
        if (e != cudaSuccess) return cuda_fail(e, "gemv occupancy query");
        occ = n > 0 ? n : 1;
        oc.occ = occ;
        oc.smem_plus1 = smem + 1;
    }
    long want = (OUT + GEMV_WARPS - 1) / GEMV_WARPS;
    long cap = (long)sm_count() * occ;
    if (ga.idx) cap = cap * ga.shard_world / ga.nslots > 1 ? cap * ga.shard_world / ga.nslots : 1;   // CTAs per slot
    const dim3 grid((unsigned)(want < cap ? want : cap), (unsigned)(ga.idx ? ga.nslots : 1));
    // every expert's base stays 16-byte aligned when Wq is, because OUT*IN/2 is a multiple of 16
    cudaError_t le = launch_pdl(kern, grid, dim3(GEMV_WARPS * 32), smem, st, xq, xs, Wq, sw, Y, IN, OUT, S, aligned(Wq, 16), ga, oa);
    if (le != cudaSuccess) return cuda_fail(le, "gemv_w4a8 launch");
    return launch_status("gemv_w4a8");
}

template <int MT, int U, typename ST>
inline int launch_gemv_dp4a_t(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y,
                              int IN, int OUT, int S, cudaStream_t st, const GroupedArgs &ga, const OutArgs &oa) {
    if (oa.peers) return launch_gemv_dp4a_p<MT, U, ST, true>(xq, xs, Wq, sw, Y, IN, OUT, S, st, ga, oa);
    return launch_gemv_dp4a_p<MT, U, ST, false>(xq, xs, Wq, sw, Y, IN, OUT, S, st, ga, oa);
}

template <int MT, typename ST>
inline int launch_gemv_dp4a_u(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y,
                              int IN, int OUT, int S, cudaStream_t st, const GroupedArgs &ga = GroupedArgs(),
                              const OutArgs &oa = OutArgs()) {
    const int nslots = (IN / QBLK + 31) / 32;
    // Loads in flight per lane: the whole row when it has at most 5 slots, else the divisor of the slot
    // count that wastes no predicated slot (5 for K = 15360), else 4.
    int u = nslots <= 5 ? nslots : (nslots % 5 == 0 ? 5 : (nslots % 3 == 0 ? 3 : 4));
    switch (u) {
        case 1: return launch_gemv_dp4a_t<MT, 1, ST>(xq, xs, Wq, sw, Y, IN, OUT, S, st, ga, oa);
        case 2: return launch_gemv_dp4a_t<MT, 2, ST>(xq, xs, Wq, sw, Y, IN, OUT, S, st, ga, oa);
        case 3: return launch_gemv_dp4a_t<MT, 3, ST>(xq, xs, Wq, sw, Y, IN, OUT, S, st, ga, oa);
        case 4: return launch_gemv_dp4a_t<MT, 4, ST>(xq, xs, Wq, sw, Y, IN, OUT, S, st, ga, oa);
        default: return launch_gemv_dp4a_t<MT, 5, ST>(xq, xs, Wq, sw, Y, IN, OUT, S, st, ga, oa);
    }
}

template <typename ST>
inline int launch_gemv_st(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y,
                          int IN, int OUT, int S, cudaStream_t st, const OutArgs &oa_in) {
    const int nb = IN / QBLK;
    // Rows beyond GEMV_MT_MAX go in further passes over the weights (which then come from L2).
    OutArgs oa = oa_in;
    const size_t y_off0 = oa.y_off;
    for (int s0 = 0; s0 < S; s0 += GEMV_MT_MAX) {
        const int s = S - s0 < GEMV_MT_MAX ? S - s0 : GEMV_MT_MAX;
        if (oa.peers) oa.y_off = y_off0 + (size_t)s0 * oa.ld * sizeof(float);
        const int8_t *xq_p = xq + (size_t)s0 * IN;
        const float *xs_p = xs + (size_t)s0 * nb;
        float *y_p = Y + (size_t)s0 * OUT;
        int rc;
        switch (s) {
            case 1: rc = launch_gemv_dp4a_u<1, ST>(xq_p, xs_p, Wq, sw, y_p, IN, OUT, s, st, GroupedArgs(), oa); break;
            case 2: rc = launch_gemv_dp4a_u<2, ST>(xq_p, xs_p, Wq, sw, y_p, IN, OUT, s, st, GroupedArgs(), oa); break;
            case 3: rc = launch_gemv_dp4a_u<3, ST>(xq_p, xs_p, Wq, sw, y_p, IN, OUT, s, st, GroupedArgs(), oa); break;
            default: rc = launch_gemv_dp4a_u<4, ST>(xq_p, xs_p, Wq, sw, y_p, IN, OUT, s, st, GroupedArgs(), oa); break;
        }
        if (rc != W4A8_OK) return rc;
    }
    return W4A8_OK;
}

template <typename ST>
inline int launch_gemv_short(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int IN, int OUT,
                             cudaStream_t st, const GroupedArgs &ga);

inline int launch_gemv(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                       int IN, int OUT, int S, int scale_dtype, cudaStream_t st, const OutArgs &oa = OutArgs()) {
    if (S == 0 || OUT == 0) return W4A8_OK;
    if (S == 1 && IN <= 32 * QBLK && !oa.peers) {        // one short row: the R-rows-per-warp kernel (same bits)
        if (scale_dtype == 1) return launch_gemv_short<__half>(xq, xs, Wq, (const __half *)sw, Y, IN, OUT, st, GroupedArgs());
        return launch_gemv_short<float>(xq, xs, Wq, (const float *)sw, Y, IN, OUT, st, GroupedArgs());
    }
    if (scale_dtype == 1) return launch_gemv_st<__half>(xq, xs, Wq, (const __half *)sw, Y, IN, OUT, S, st, oa);
    return launch_gemv_st<float>(xq, xs, Wq, (const float *)sw, Y, IN, OUT, S, st, oa);
}

// ---- short rows (K <= 2048: NG = one or two groups per lane), one activation row, optional expert grouping --------
// On rows this short the persistent kernel above keeps only two batches of 16-byte loads per lane in flight and spends
// most of its instructions on its item bookkeeping (194 warp instructions per 64-group row of the expert gate|up
// projection, 2.3 TB/s on the 768-wide down projection).  Here a warp takes R consecutive output rows at a time — lane l
// loads groups l, l + 32, ... of each of them, with the next R rows' loads issued before the current ones are used — so
// 2 R NG loads are in flight per lane.  Same arithmetic per row as the persistent kernel (lane l chains
// acc = fma((xs*sw)/16, (float)(16*D), acc) over its groups in ascending order from 0, then the shfl_down tree):
// identical bits.
template <int R, int NG, typename ST>
__global__ void __launch_bounds__(SHORT_WARPS * 32) gemv_w4a8_short_kernel(
    const int8_t *__restrict__ xq, const float *__restrict__ xs, const uint8_t *__restrict__ Wq,
    const ST *__restrict__ sw, float *__restrict__ Y, int IN, int OUT, bool w_a16, GroupedArgs ga) {
    const int nb = IN / QBLK;                                       // <= 32 * NG
    __shared__ __align__(16) uint32_t xrow_s[NG * 32 * 8];          // src_mode 1: the quantized activation row
    __shared__ float xs_s[NG * 32];
    int row = 0;
    if (ga.idx) {                                                   // blockIdx.y = slot (see the persistent kernel)
        const int slot = blockIdx.y;
        pdl_wait();   // the routing indices are written by an earlier kernel of the stream: wait before reading them
        const int e = ga.idx[slot] - ga.expert_base;
        if (e < 0 || e >= ga.num_experts) return;
        row = ga.x_per_slot ? slot : slot / ga.topk;
        xq += (size_t)row * IN;
        xs += (size_t)row * nb;
        Wq += (size_t)e * ((size_t)OUT * (IN / 2));
        sw += (size_t)e * ((size_t)OUT * nb);
        Y += (size_t)slot * OUT;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t wpitch = (size_t)(IN / 2);
    const bool fused = ga.src_mode == 1;
    // units of R rows, dealt round-robin to the warps of the grid
    const int units = (OUT + R - 1) / R;
    const int gw = blockIdx.x * SHORT_WARPS + warp, nw = gridDim.x * SHORT_WARPS;
    bool live[NG];
#pragma unroll
    for (int g = 0; g < NG; g++) live[g] = lane + 32 * g < nb;
    uint4 wa[R * NG], wb[R * NG];
    float sa[R * NG], sb_[R * NG];
    auto load = [&](int unit, uint4 (&w)[R * NG], float (&sc)[R * NG]) {
#pragma unroll
        for (int i = 0; i < R; i++) {
            const int r = unit * R + i;
#pragma unroll
            for (int g = 0; g < NG; g++) {
                const int b = lane + 32 * g;
                if (live[g] && r < OUT) { w[i * NG + g] = ldg_w16(Wq + (size_t)r * wpitch + 16 * b, w_a16); sc[i * NG + g] = load_scale(sw + (size_t)r * nb, b); }
                else { w[i * NG + g] = make_uint4(0, 0, 0, 0); sc[i * NG + g] = 0.f; }
            }
        }
    };
    pdl_launch_dependents();
    if (gw < units) load(gw, wa, sa);                               // weights only: allowed before the dependency wait
    pdl_wait();
    if (fused) {
        // quantize_x of the token's row, every CTA of the slot for itself (IN <= 2048 floats out of L2); the values and
        // their order are quantize_x_q8_vec_kernel's
        const float4 *xr = reinterpret_cast<const float4 *>(ga.src_f32 + (size_t)row * IN);
        uint32_t *gq = blockIdx.x == 0 ? reinterpret_cast<uint32_t *>(ga.xq_out + (size_t)row * IN) : nullptr;
        float *gs = blockIdx.x == 0 ? ga.xs_out + (size_t)row * nb : nullptr;
        const int nvec = IN / 4;
        for (int i = tid; i - lane < nvec; i += SHORT_WARPS * 32) {
            const bool lv = i < nvec;
            const float4 v = lv ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            quantize_row_vec4(v, i, lv, xrow_s, xs_s, gq, gs);
        }
        __syncthreads();
    }
    // this lane's groups of the activation row (lane, lane + 32, ...), split into even / odd bytes to match unpack8_x16
    uint32_t xe[NG][4], xo[NG][4];
    float xsv[NG];
#pragma unroll
    for (int g = 0; g < NG; g++) {
#pragma unroll
        for (int i = 0; i < 4; i++) xe[g][i] = xo[g][i] = 0u;
        xsv[g] = 0.f;
        if (live[g]) {
            uint32_t v[8];
            if (fused) {
                const uint4 *src = reinterpret_cast<const uint4 *>(xrow_s + (lane + 32 * g) * 8);
                const uint4 v0 = src[0], v1 = src[1];
                v[0] = v0.x; v[1] = v0.y; v[2] = v0.z; v[3] = v0.w; v[4] = v1.x; v[5] = v1.y; v[6] = v1.z; v[7] = v1.w;
                xsv[g] = xs_s[lane + 32 * g];
            } else {
                const uint32_t *src = reinterpret_cast<const uint32_t *>(xq + (size_t)(lane + 32 * g) * QBLK);
#pragma unroll
                for (int i = 0; i < 8; i++) v[i] = src[i];
                xsv[g] = xs[lane + 32 * g];
            }
#pragma unroll
            for (int i = 0; i < 4; i++) split_even_odd(v[2 * i], v[2 * i + 1], xe[g][i], xo[g][i]);
        }
    }
    auto compute = [&](int unit, const uint4 (&w)[R * NG], const float (&sc)[R * NG]) {
        float acc[R];
#pragma unroll
        for (int i = 0; i < R; i++) {
            acc[i] = 0.f;
#pragma unroll
            for (int g = 0; g < NG; g++) {
                const uint4 wv = w[i * NG + g];
                uint32_t e0, o0, e1, o1, e2, o2, e3, o3;
                unpack8_x16(wv.x, e0, o0); unpack8_x16(wv.y, e1, o1);
                unpack8_x16(wv.z, e2, o2); unpack8_x16(wv.w, e3, o3);
                int d = __dp4a((int)xe[g][0], (int)e0, 0);
                d = __dp4a((int)xo[g][0], (int)o0, d);
                d = __dp4a((int)xe[g][1], (int)e1, d);
                d = __dp4a((int)xo[g][1], (int)o1, d);
                d = __dp4a((int)xe[g][2], (int)e2, d);
                d = __dp4a((int)xo[g][2], (int)o2, d);
                d = __dp4a((int)xe[g][3], (int)e3, d);
                d = __dp4a((int)xo[g][3], (int)o3, d);              // d = 16 * D[o,b], exact
                const float scv = (xsv[g] * sc[i * NG + g]) * 0.0625f;   // exact 1/16
                if (live[g]) acc[i] = fmaf(scv, (float)d, acc[i]);  // the persistent kernel's chain: groups lane, lane + 32, ...
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1)
#pragma unroll
            for (int i = 0; i < R; i++) acc[i] += __shfl_down_sync(0xffffffffu, acc[i], off);
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < R; i++)
                if (unit * R + i < OUT) Y[unit * R + i] = acc[i];
        }
    };
    for (int u = gw; u < units; u += 2 * nw) {
        if (u + nw < units) load(u + nw, wb, sb_);
        compute(u, wa, sa);
        if (u + nw >= units) break;
        if (u + 2 * nw < units) load(u + 2 * nw, wa, sa);
        compute(u + nw, wb, sb_);
    }
}

// ---- rows of 24 groups (K = 768, the expert down projection of benchmark configuration 5), one activation row -------
// With a lane per group the kernel above idles 8 lanes of 32 and pays a 5-level shuffle tree per row: 85 warp
// instructions per 480-byte row, 2.3 TB/s.  Rows of 24 groups are contiguous in memory (384 bytes of nibbles, 24 scales),
// so here a warp walks the matrix as a flat sequence of groups: a tile is 4 rows = 96 groups = three fully coalesced
// 512-byte loads (+ three 128-byte scale loads), lane l of load j holding flat group 32 j + l, i.e. group (32 j + l) % 24
// of row (32 j + l) / 24.  The per-group products go through shared memory and eight lanes per row add them in the
// order of the shfl_down tree over lanes 0..23 of the lane-per-group kernel (lanes 24..31 there carry +0):
// ((v[i] + v[i+16]) + (v[i+8] + 0)) for i < 8, then the offsets 4, 2, 1.  Same products, same order: identical bits.
template <typename ST>
__global__ void __launch_bounds__(GEMV_WARPS * 32) gemv_w4a8_flat24_kernel(
    const int8_t *__restrict__ xq, const float *__restrict__ xs, const uint8_t *__restrict__ Wq,
    const ST *__restrict__ sw, float *__restrict__ Y, int OUT, GroupedArgs ga) {
    constexpr int NB = 24, TR = 4, TL = 3;                          // groups per row, rows and loads per tile
    __shared__ float part[GEMV_WARPS][2][TR * NB];
    __shared__ __align__(16) uint32_t xrow_s[NB * 8];               // src_mode 2: the quantized activation row
    __shared__ float xs_s[NB];
    const int slot = blockIdx.y;
    if (ga.idx) {                                                   // blockIdx.y = slot (see the persistent kernel)
        pdl_wait();   // the routing indices are written by an earlier kernel of the stream: wait before reading them
        const int e = ga.idx[slot] - ga.expert_base;
        if (e < 0 || e >= ga.num_experts) return;
        const int row = ga.x_per_slot ? slot : slot / ga.topk;
        xq += (size_t)row * (NB * QBLK);
        xs += (size_t)row * NB;
        Wq += (size_t)e * ((size_t)OUT * (NB * 16));
        sw += (size_t)e * ((size_t)OUT * NB);
        Y += (size_t)slot * OUT;
    }
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int tiles = (OUT + TR - 1) / TR, ngroups = OUT * NB;
    const int gw = blockIdx.x * GEMV_WARPS + warp, nw = gridDim.x * GEMV_WARPS;
    uint4 wa[TL], wb[TL];
    float sa[TL], sb_[TL];
    auto load = [&](int tile, uint4 (&w)[TL], float (&sc)[TL]) {
#pragma unroll
        for (int j = 0; j < TL; j++) {
            const int f = tile * (TR * NB) + 32 * j + lane;
            if (f < ngroups) { w[j] = __ldcs(reinterpret_cast<const uint4 *>(Wq) + f); sc[j] = load_scale(sw, f); }
            else { w[j] = make_uint4(0, 0, 0, 0); sc[j] = 0.f; }
        }
    };
    pdl_launch_dependents();
    if (gw < tiles) load(gw, wa, sa);                               // weights only: allowed before the dependency wait
    pdl_wait();
    const bool fused = ga.src_mode == 2;
    if (fused) {
        // activation of the slot's gate | up row and quantize_x of the result, every CTA of the slot for itself (1536 floats
        // out of L2); the values and their order are glu_quantize_kernel's
        const float4 *G = reinterpret_cast<const float4 *>(ga.src_f32 + (size_t)slot * (2 * NB * QBLK)), *U = G + NB * 8;
        uint32_t *gq = blockIdx.x == 0 ? reinterpret_cast<uint32_t *>(ga.xq_out + (size_t)slot * (NB * QBLK)) : nullptr;
        float *gs = blockIdx.x == 0 ? ga.xs_out + (size_t)slot * NB : nullptr;
        const bool lv = tid < NB * 8;
        float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lv) {
            const float4 g = G[tid], u = U[tid];
            if (ga.act == 0) y = make_float4(glu_value<0>(g.x, u.x), glu_value<0>(g.y, u.y), glu_value<0>(g.z, u.z), glu_value<0>(g.w, u.w));
            else y = make_float4(glu_value<1>(g.x, u.x), glu_value<1>(g.y, u.y), glu_value<1>(g.z, u.z), glu_value<1>(g.w, u.w));
        }
        quantize_row_vec4(y, tid, lv, xrow_s, xs_s, gq, gs);
        __syncthreads();
    }
    // the three activation groups a lane meets (the pattern repeats every tile), split into even / odd bytes and kept
    // in shared memory as two planes of 16-byte words indexed [j][lane] (conflict-free); warp j fills plane set j
    __shared__ uint4 xpat[TL][2][32];
    __shared__ float xspat[TL][32];
    if (warp < TL) {
        const int b = (32 * warp + lane) % NB;
        const uint4 *src = fused ? reinterpret_cast<const uint4 *>(xrow_s + b * 8) : reinterpret_cast<const uint4 *>(xq + (size_t)b * QBLK);
        const uint4 v0 = src[0], v1 = src[1];
        uint4 p0, p1;
        split_even_odd(v0.x, v0.y, p0.x, p0.y);
        split_even_odd(v0.z, v0.w, p0.z, p0.w);
        split_even_odd(v1.x, v1.y, p1.x, p1.y);
        split_even_odd(v1.z, v1.w, p1.z, p1.w);
        xpat[warp][0][lane] = p0;
        xpat[warp][1][lane] = p1;
        xspat[warp][lane] = fused ? xs_s[b] : xs[b];
    }
    __syncthreads();
    int parity = 0;
    auto compute = [&](int tile, const uint4 (&w)[TL], const float (&sc)[TL]) {
        float *pp = part[warp][parity];
        parity ^= 1;
#pragma unroll
        for (int j = 0; j < TL; j++) {
            uint32_t e0, o0, e1, o1, e2, o2, e3, o3;
            unpack8_x16(w[j].x, e0, o0); unpack8_x16(w[j].y, e1, o1);
            unpack8_x16(w[j].z, e2, o2); unpack8_x16(w[j].w, e3, o3);
            const uint4 p0 = xpat[j][0][lane], p1 = xpat[j][1][lane];
            const float xsj = xspat[j][lane];
            int d = __dp4a((int)p0.x, (int)e0, 0);
            d = __dp4a((int)p0.y, (int)o0, d);
            d = __dp4a((int)p0.z, (int)e1, d);
            d = __dp4a((int)p0.w, (int)o1, d);
            d = __dp4a((int)p1.x, (int)e2, d);
            d = __dp4a((int)p1.y, (int)o2, d);
            d = __dp4a((int)p1.z, (int)e3, d);
            d = __dp4a((int)p1.w, (int)o3, d);                      // d = 16 * D[o,b], exact
            const float scv = (xsj * sc[j]) * 0.0625f;              // exact 1/16
            pp[32 * j + lane] = fmaf(scv, (float)d, 0.f);
        }
        __syncwarp();
        // lane = 8 r + i adds groups i, i + 16 and i + 8 of row r; a second buffer (parity) spares the barrier that
        // would otherwise have to keep the next tile's stores behind these loads
        const float *v = pp + (lane >> 3) * NB + (lane & 7);
        float a = __fadd_rn(__fadd_rn(v[0], v[16]), __fadd_rn(v[8], 0.f));
        a = __fadd_rn(a, __shfl_down_sync(0xffffffffu, a, 4));
        a = __fadd_rn(a, __shfl_down_sync(0xffffffffu, a, 2));
        a = __fadd_rn(a, __shfl_down_sync(0xffffffffu, a, 1));
        const int r = tile * TR + (lane >> 3);
        if ((lane & 7) == 0 && r < OUT) Y[r] = a;
    };
    for (int u = gw; u < tiles; u += 2 * nw) {
        if (u + nw < tiles) load(u + nw, wb, sb_);
        compute(u, wa, sa);
        if (u + nw >= tiles) break;
        if (u + 2 * nw < tiles) load(u + 2 * nw, wa, sa);
        compute(u + nw, wb, sb_);
    }
}

template <typename ST>
inline int launch_gemv_flat24(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int OUT,
                              cudaStream_t st, const GroupedArgs &ga) {
    auto kern = gemv_w4a8_flat24_kernel<ST>;
    static PerDevice<int> occ_dev;
    int &occ = occ_dev.get();
    if (occ == 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, GEMV_WARPS * 32, 0);
        if (e != cudaSuccess) return cuda_fail(e, "gemv_flat24 occupancy query");
        occ = n > 0 ? n : 1;
    }
    const long tiles = (OUT + 3) / 4;
    long want = (tiles + GEMV_WARPS - 1) / GEMV_WARPS, cap = (long)sm_count() * occ;
    if (ga.idx) cap = cap * ga.shard_world / ga.nslots > 1 ? cap * ga.shard_world / ga.nslots : 1;   // CTAs per slot
    const dim3 grid((unsigned)(want < cap ? want : cap), (unsigned)(ga.idx ? ga.nslots : 1));
    cudaError_t le = launch_pdl(kern, grid, dim3(GEMV_WARPS * 32), 0, st, xq, xs, Wq, sw, Y, OUT, ga);
    if (le != cudaSuccess) return cuda_fail(le, "gemv_w4a8_flat24 launch");
    return launch_status("gemv_w4a8_flat24");
}

template <int R, int NG, typename ST>
inline int launch_gemv_short_rn(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int IN, int OUT,
                                cudaStream_t st, const GroupedArgs &ga) {
    auto kern = gemv_w4a8_short_kernel<R, NG, ST>;
    static PerDevice<int> occ_dev;
    int &occ = occ_dev.get();
    if (occ == 0) {
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, SHORT_WARPS * 32, 0);
        if (e != cudaSuccess) return cuda_fail(e, "gemv_short occupancy query");
        occ = n > 0 ? n : 1;
    }
    const long units = (OUT + R - 1) / R;
    long want = (units + SHORT_WARPS - 1) / SHORT_WARPS, cap = (long)sm_count() * occ;
    if (ga.idx) cap = cap * ga.shard_world / ga.nslots > 1 ? cap * ga.shard_world / ga.nslots : 1;   // CTAs per slot
    const dim3 grid((unsigned)(want < cap ? want : cap), (unsigned)(ga.idx ? ga.nslots : 1));
    cudaError_t le = launch_pdl(kern, grid, dim3(SHORT_WARPS * 32), 0, st, xq, xs, Wq, sw, Y, IN, OUT, aligned(Wq, 16), ga);
    if (le != cudaSuccess) return cuda_fail(le, "gemv_w4a8_short launch");
    return launch_status("gemv_w4a8_short");
}

// K <= 2048.  Rows of at most 32 groups take four rows per warp step; rows of 33..64 groups two rows with two groups per
// lane (the same eight loads in flight per lane).
template <typename ST>
inline int launch_gemv_short(const int8_t *xq, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int IN, int OUT,
                             cudaStream_t st, const GroupedArgs &ga) {
    // rows of exactly 24 groups, 16-byte aligned everywhere: the flat-group kernel (the tile loop indexes with int)
    if (ga.src_mode != 1 && IN == 24 * QBLK && aligned(Wq, 16) && aligned(xq, 16) && (long)OUT * 24 < (1L << 30))
        return launch_gemv_flat24<ST>(xq, xs, Wq, sw, Y, OUT, st, ga);
    if (ga.src_mode == 2) return fail(W4A8_ERR_UNSUPPORTED, "gemv_short: the fused activation prologue needs rows of 24 groups");
    if (IN > 32 * QBLK) return launch_gemv_short_rn<2, 2, ST>(xq, xs, Wq, sw, Y, IN, OUT, st, ga);
    return launch_gemv_short_rn<4, 1, ST>(xq, xs, Wq, sw, Y, IN, OUT, st, ga);
}

// Grouped experts: one launch, grid.y = slots, each slot one activation row against its expert.  fused (optional): the
// src_mode / act / src_f32 / xq_out / xs_out fields of a GroupedArgs, for K <= 2048 only (see the struct).
inline int launch_moe_gemv(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, const int32_t *idx,
                           float *Y, int nslots, int topk, int x_per_slot, int N, int K, int num_experts,
                           int scale_dtype, cudaStream_t st, int expert_base = 0, int shard_world = 1,
                           const GroupedArgs *fused = nullptr) {
    if (nslots == 0 || N == 0) return W4A8_OK;
    if (nslots > 65535) return fail(W4A8_ERR_UNSUPPORTED, "moe_gemv: at most 65535 slots per launch (got %d)", nslots);
    GroupedArgs ga;
    if (fused) ga = *fused;
    ga.idx = idx; ga.topk = topk; ga.x_per_slot = x_per_slot; ga.num_experts = num_experts; ga.nslots = nslots;
    ga.expert_base = expert_base;
    ga.shard_world = shard_world < 1 ? 1 : shard_world;
    if (K <= 64 * QBLK) {                                           // short rows: the R-rows-per-warp kernels
        if (scale_dtype == 1) return launch_gemv_short<__half>(xq, xs, Wq, (const __half *)sw, Y, K, N, st, ga);
        return launch_gemv_short<float>(xq, xs, Wq, (const float *)sw, Y, K, N, st, ga);
    }
    if (ga.src_mode != 0) return fail(W4A8_ERR_UNSUPPORTED, "moe_gemv: fused prologues need K <= 2048");
    if (scale_dtype == 1) return launch_gemv_dp4a_u<1, __half>(xq, xs, Wq, (const __half *)sw, Y, K, N, 1, st, ga);
    return launch_gemv_dp4a_u<1, float>(xq, xs, Wq, (const float *)sw, Y, K, N, 1, st, ga);
}

}  // namespace w4a8
