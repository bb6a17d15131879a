// Routed-expert MLP block in W4A8: the four launches of the reference's fused MoE path (models/moe_block.cuh:45-52:
// grouped gate_up, swiglu, grouped down, fixed-order reduce — kernels/moe_fused.cuh:14-76) with the expert products
// done in W4A8 arithmetic (activations quantized per 32-element block like every other matmul on this path; the
// reference's own expert kernels are W4A32).  Kept from the reference: the flat expert tensors
// experts_gate_up[E][2*MI][H] (rows [0,MI) gate, [MI,2*MI) up, kernels/moe_fused.cuh:40-42) and experts_down[E][H][MI]
// (runtime/weights_qwen.cu:62-63), slot = token*topk + k with the expert id idx[slot] read on the device, the router
// weight applied to the slot's down output, and the combine in ascending k without atomics (kernels/moe_fused.cuh:68-76).
//
// Few slots (decode): one grouped GEMV launch per projection, one CTA column per slot.  Many slots (prefill): the slots
// are sorted by expert on the device and both projections run as grouped GEMMs on the tensor cores — work unit =
// (expert, tile of up to 64 of its rows) x 128 output columns, every expert's weights streamed once.
// An expert shard (experts [expert_base, expert_base + experts) on this rank) computes only the slots routed to its
// experts; the slots' down outputs are then sent to every rank's arena (moe_push_rows_kernel) and every rank combines.
#pragma once
#include "common.cuh"
#include "fused_quantize.cuh"
#include "gemm_w4a8_tc.cuh"
#include "gemv_w4a8.cuh"
#include "peer_allgather.cuh"
#include "quantize_x.cuh"

namespace w4a8 {
namespace moe {

constexpr int MAX_EXPERTS = 1024;
constexpr int TILE_ROWS = gemm::BNG;   // rows per item of the grouped GEMM = its accumulator's columns

// Byte offsets of the block's intermediates inside the caller's workspace (all 256-byte aligned).
struct Layout {
    size_t perm, pos, offsets, items, num_items;   // sort: sorted row -> slot, slot -> sorted row (-1: not on this rank),
                                                   // first sorted row of every local expert [experts + 1], item list, its length
    size_t xq, xs;                                 // quantized tokens [S][H], [S][H/32]
    size_t xq_g, xs_g;                             // the same rows gathered per sorted row [nslots][H] (GEMM path)
    size_t gu;                                     // gate|up outputs [nslots][2*MI] fp32 (GEMM path: sorted rows; GEMV path: slots)
    size_t xq_h, xs_h;                             // quantized hidden activations [nslots][MI], [nslots][MI/32] (same row order)
    size_t sout;                                   // down outputs [nslots][H] fp32 (same row order), router weight not applied yet
    size_t bytes;
    int max_items;
};
inline Layout layout_for(int S, int topk, int H, int MI, int experts) {
    Layout l;
    const size_t nslots = (size_t)S * topk;
    size_t o = 0;
    auto take = [&](size_t n) { const size_t at = o; o += (n + 255) & ~(size_t)255; return at; };
    l.max_items = experts + (int)(nslots / TILE_ROWS) + 1;
    l.perm = take(nslots * 4);
    l.pos = take(nslots * 4);
    l.offsets = take(((size_t)experts + 1) * 4);
    l.items = take((size_t)l.max_items * 16);
    l.num_items = take(4);
    l.xq = take((size_t)S * H);
    l.xs = take((size_t)S * (H / QBLK) * 4);
    l.xq_g = take(nslots * H);
    l.xs_g = take(nslots * (H / QBLK) * 4);
    l.gu = take(nslots * 2 * MI * 4);
    l.xq_h = take(nslots * MI);
    l.xs_h = take(nslots * (MI / QBLK) * 4);
    l.sout = take(nslots * H * 4);
    l.bytes = o;
    return l;
}

// One CTA of 1024 threads.  Stable counting sort of the slots by local expert id (idx[slot] - expert_base; ids outside
// [0, experts) belong to another rank or are invalid and get pos = -1), and the item list of the grouped GEMM.
//   1. every warp owns a contiguous segment of the slots and counts its experts (per-warp histogram rows in shared
//      memory when experts <= FAST_EXPERTS, else one shared histogram);
//   2. warp 0 scans the expert totals 32 at a time (offsets, number of 64-row tiles) and writes the item list;
//   3. thread e turns column e of the per-warp histograms into the warps' first positions for expert e;
//   4. every warp walks its segment 32 slots at a time: a slot's position = its warp's running position for the
//      expert + its rank among the equal ids of the 32 (match_any), so an expert's rows keep the slots' order.
// More than FAST_EXPERTS experts: step 4 is done expert by expert (a warp takes an expert and walks all slots).
__global__ void __launch_bounds__(1024) moe_sort_kernel(const int32_t *__restrict__ idx, int nslots, int expert_base, int experts,
                                                        int *__restrict__ perm, int *__restrict__ pos, int *__restrict__ offsets,
                                                        int4 *__restrict__ items, int *__restrict__ num_items) {
    constexpr int FAST_EXPERTS = 256, NW = 32;
    __shared__ int cnt[MAX_EXPERTS];
    __shared__ int off[MAX_EXPERTS + 1];
    __shared__ int wpos[NW][FAST_EXPERTS];     // fast path: per-warp counts, then per-warp running positions
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool fast = experts <= FAST_EXPERTS;
    const int seg = ((nslots + NW - 1) / NW + 31) & ~31;             // slots per warp, a multiple of 32
    const int s_begin = warp * seg, s_end = min(nslots, s_begin + seg);
    for (int e = tid; e < experts; e += blockDim.x) cnt[e] = 0;
    if (fast)
        for (int i = tid; i < NW * FAST_EXPERTS; i += blockDim.x) (&wpos[0][0])[i] = 0;
    __syncthreads();
    for (int s = s_begin + lane; s < s_end; s += 32) {
        const int e = idx[s] - expert_base;
        if (e >= 0 && e < experts) {
            atomicAdd(&cnt[e], 1);
            if (fast) atomicAdd(&wpos[warp][e], 1);
        } else {
            pos[s] = -1;
        }
    }
    __syncthreads();
    if (warp == 0) {
        int run = 0, n = 0;
        for (int e0 = 0; e0 < experts; e0 += 32) {
            const int e = e0 + lane;
            const int c = e < experts ? cnt[e] : 0;
            const int t = (c + TILE_ROWS - 1) / TILE_ROWS;
            int ic = c, it = t;                                        // inclusive scans over the 32 experts
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int uc = __shfl_up_sync(0xffffffffu, ic, d), ut = __shfl_up_sync(0xffffffffu, it, d);
                if (lane >= d) { ic += uc; it += ut; }
            }
            const int first = run + ic - c, item0 = n + it - t;
            if (e < experts) {
                off[e] = first;
                offsets[e] = first;
                for (int k = 0; k < t; k++) items[item0 + k] = make_int4(e, first + k * TILE_ROWS, min(TILE_ROWS, c - k * TILE_ROWS), 0);
            }
            run += __shfl_sync(0xffffffffu, ic, 31);
            n += __shfl_sync(0xffffffffu, it, 31);
        }
        if (lane == 0) {
            off[experts] = run;
            offsets[experts] = run;
            *num_items = n;
        }
    }
    __syncthreads();
    if (fast) {
        for (int e = tid; e < experts; e += blockDim.x) {               // counts -> first positions, warps in order
            int p = off[e];
            for (int w = 0; w < NW; w++) { const int c = wpos[w][e]; wpos[w][e] = p; p += c; }
        }
        __syncthreads();
        for (int s0 = s_begin; s0 < s_end; s0 += 32) {                  // uniform per warp
            const int s = s0 + lane;
            int e = s < s_end ? idx[s] - expert_base : -1;
            if (e < 0 || e >= experts) e = -1;
            const unsigned same = __match_any_sync(0xffffffffu, e);
            if (e >= 0) {
                const int p = wpos[warp][e] + __popc(same & ((1u << lane) - 1u));
                perm[p] = s;
                pos[s] = p;
            }
            __syncwarp();
            if (e >= 0 && lane == 31 - __clz(same)) wpos[warp][e] += __popc(same);   // the last of the equal ids moves the position on
            __syncwarp();
        }
        return;
    }
    // many experts: a warp takes an expert and walks all slots 32 at a time
    for (int e = warp; e < experts; e += NW) {
        if (cnt[e] == 0) continue;
        int placed = 0;
        for (int s0 = 0; s0 < nslots; s0 += 32) {
            const int s = s0 + lane;
            const bool mine = s < nslots && idx[s] - expert_base == e;
            const unsigned m = __ballot_sync(0xffffffffu, mine);
            if (mine) {
                const int p = off[e] + placed + __popc(m & ((1u << lane) - 1u));
                perm[p] = s;
                pos[s] = p;
            }
            placed += __popc(m);
        }
    }
}

// Sorted row p < offsets[experts] gets the quantized activations of its token perm[p] / topk.
__global__ void __launch_bounds__(128) moe_gather_rows_kernel(const int8_t *__restrict__ xq, const float *__restrict__ xs,
                                                              const int *__restrict__ perm, const int *__restrict__ count, int topk, int K,
                                                              int8_t *__restrict__ xq_g, float *__restrict__ xs_g) {
    const int n = *count, nb = K / QBLK;
    for (int p = blockIdx.x; p < n; p += gridDim.x) {
        const int tok = perm[p] / topk;
        const uint4 *src = reinterpret_cast<const uint4 *>(xq + (size_t)tok * K);
        uint4 *dst = reinterpret_cast<uint4 *>(xq_g + (size_t)p * K);
        for (int i = threadIdx.x; i < K / 16; i += blockDim.x) dst[i] = src[i];
        for (int i = threadIdx.x; i < nb; i += blockDim.x) xs_g[(size_t)p * nb + i] = xs[(size_t)tok * nb + i];
    }
}

// out[b, o] = sum over k ascending of dw[b*topk + k] * Sout[row(b*topk + k), o], starting from 0: the values and the
// order of kernels/moe_fused.cuh:64 (router weight times the slot's down output, one rounding) and :68-76.
// pos != nullptr: Sout is in sorted-row order, row(slot) = pos[slot] (slots with pos < 0 contribute nothing);
// pos == nullptr: Sout is in slot order.  H a multiple of 4.
__global__ void __launch_bounds__(256) moe_combine_kernel(const float4 *__restrict__ Sout, const int *__restrict__ pos, const float *__restrict__ dw,
                                                          float4 *__restrict__ out, int H4, int topk, long total /* = S * H4 */) {
    const long stride = (long)gridDim.x * blockDim.x;
    pdl_launch_dependents();
    pdl_wait();   // the down outputs come from the kernel before this one
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long b = i / H4;
        const int o = (int)(i - b * H4);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < topk; k++) {
            const long slot = b * topk + k;
            const long row = pos ? pos[slot] : slot;
            if (row < 0) continue;
            const float w = dw[slot];
            const float4 v = Sout[row * H4 + o];
            acc.x = __fadd_rn(acc.x, __fmul_rn(w, v.x));
            acc.y = __fadd_rn(acc.y, __fmul_rn(w, v.y));
            acc.z = __fadd_rn(acc.z, __fmul_rn(w, v.z));
            acc.w = __fadd_rn(acc.w, __fmul_rn(w, v.w));
        }
        out[i] = acc;
    }
}

// Expert shard: the down outputs of this rank's slots (sorted rows p < *count of `src`, or — grouped GEMV path, no sort —
// the slots whose expert id is local) go to row `slot` of the slot-ordered buffer at y_off in EVERY rank's arena, 16-byte stores, consecutive lanes
// on consecutive pieces of a row; then one system fence per CTA, the last CTA publishes `epoch` and (wait_limit > 0)
// waits for every rank's flag.
__global__ void __launch_bounds__(256) moe_push_rows_kernel(const PeerDesc *p, const float4 *__restrict__ src, int sorted,
                                                            const int *__restrict__ perm, const int *__restrict__ count, int H4, size_t y_off,
                                                            unsigned int epoch, long long wait_limit, const int32_t *__restrict__ idx,
                                                            int nslots, int expert_base, int experts) {
    // perm != nullptr: this rank's rows are sorted rows 0 .. *count - 1 (slot perm[r]); perm == nullptr (grouped GEMV
    // path, src in slot order): every slot whose expert id lies in this rank's range
    const int n = perm ? *count : nslots, world = p->world;
    for (int r = blockIdx.x; r < n; r += gridDim.x) {
        int slot = r;
        if (perm) slot = perm[r];
        else { const int e = idx[r] - expert_base; if (e < 0 || e >= experts) continue; }
        const float4 *s = src + (size_t)(sorted ? r : slot) * H4;
        for (int i = threadIdx.x; i < H4; i += blockDim.x) {
            const float4 v = s[i];
            for (int k = 0; k < world; k++) reinterpret_cast<float4 *>(p->base[k] + y_off)[(size_t)slot * H4 + i] = v;
        }
    }
    __syncthreads();
    __shared__ unsigned int s_last;
    if (threadIdx.x == 0) {
        __threadfence_system();
        s_last = (atomicAdd(p->counter, 1u) == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) {
        *p->counter = 0u;
        publish_flags(p, epoch);
    }
    if (wait_limit > 0 && threadIdx.x < 32) wait_flags(p, epoch, wait_limit);
}

// Expert shard, few slots (the decode form): the row exchange with tagged slots instead of fences and flags
// (peer_allgather.cuh).  Every element of a local slot's down output goes to the slot buffer of every other arena as one
// 8-byte store {value, tag of the step}; the combine reads local slots from this rank's own Sout and polls the slot
// buffer for the others (bounded; error 0x209).  Needs nslots * H <= LL_MAX_SLOTS.
__global__ void __launch_bounds__(256) moe_push_rows_ll_kernel(const PeerDesc *p, const float *__restrict__ sout, const int32_t *__restrict__ idx,
                                                               int nslots, int H, int expert_base, int experts, unsigned int epoch) {
    const unsigned int e = *p->epoch_base + epoch;
    const unsigned long long tag = (unsigned long long)ll_tag(e) << 32;
    const size_t off = p->ll_off + (size_t)(e & 1u) * LL_BUF_BYTES;
    const int world = p->world, rank = p->rank;
    for (int r = blockIdx.x; r < nslots; r += gridDim.x) {
        const int le = idx[r] - expert_base;
        if (le < 0 || le >= experts) continue;                  // another rank's slot
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const unsigned long long pk = tag | (unsigned long long)__float_as_uint(sout[(size_t)r * H + i]);
            for (int k = 0; k < world; k++)
                if (k != rank) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p->base[k] + off + ((size_t)r * H + i) * 8), "l"(pk) : "memory");
        }
    }
}
__global__ void __launch_bounds__(256) moe_combine_ll_kernel(const PeerDesc *p, const float *__restrict__ sout, const int32_t *__restrict__ idx,
                                                             const float *__restrict__ dw, float *__restrict__ out, int H, int topk, long total,
                                                             int expert_base, int experts, unsigned int epoch, long long limit) {
    const unsigned int e = *p->epoch_base + epoch, tag = ll_tag(e);
    const unsigned long long *slots = reinterpret_cast<const unsigned long long *>(p->base[p->rank] + p->ll_off + (size_t)(e & 1u) * LL_BUF_BYTES);
    const long stride = (long)gridDim.x * blockDim.x;
    bool gave_up = false;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long b = i / H;
        const int o = (int)(i - b * H);
        float acc = 0.f;
        for (int k = 0; k < topk; k++) {
            const long slot = b * topk + k;
            const int le = idx[slot] - expert_base;
            float v = 0.f;
            if (le >= 0 && le < experts) {
                v = sout[slot * H + o];
            } else {
                const long long t0 = clock64();
                for (;;) {
                    unsigned long long x;
                    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(x) : "l"(slots + slot * H + o) : "memory");
                    if ((unsigned int)(x >> 32) == tag) { v = __uint_as_float((unsigned int)x); break; }
                    if (gave_up) break;
                    if (clock64() - t0 > limit) { dev_set_error(0x209u); gave_up = true; break; }
                }
            }
            acc = __fadd_rn(acc, __fmul_rn(dw[slot], v));
        }
        out[i] = acc;
    }
}

struct BlockArgs {
    const float *n2 = nullptr;                                   // [S][H] fp32 (post-attention norm output)
    const uint8_t *gu_wq = nullptr, *dn_wq = nullptr;            // this rank's experts: [experts][2*MI][H/2], [experts][H][MI/2]
    const void *gu_sc = nullptr, *dn_sc = nullptr;
    const int32_t *idx = nullptr;                                // [S*topk] global expert ids (device)
    const float *dw = nullptr;                                   // [S*topk] router weights (device)
    float *out = nullptr;                                        // [S][H]
    int S = 0, topk = 0, H = 0, MI = 0, expert_base = 0, experts = 0, scale_dtype = 0, act = 0;
    int kernel = 0;                                              // 0 auto, 1 grouped GEMV, 2 grouped GEMM
    int world = 1;                                               // ranks the experts are split over (sizes the grouped GEMV's grid)
    unsigned char *ws = nullptr;
    const PeerDesc *peers = nullptr;                             // expert shard: every arena's slot-ordered Sout at sout_off
    unsigned char *arena_base = nullptr;
    size_t sout_off = 0;
    unsigned int epoch = 0;
    long long wait_limit = 0;
    int phase = 0;                                               // expert shard: 0 whole block, 1 up to the publish (no wait, no combine),
                                                                 //               2 wait + combine only
};

constexpr int GEMV_MAX_SLOTS = 128;   // auto: up to this many slots one CTA column per slot, above it the sorted GEMM

struct Buffers {
    int *perm, *pos, *offsets, *num_items;
    int4 *items;
    int8_t *xq, *xq_g, *xq_h;
    float *xs, *xs_g, *xs_h, *gu, *sout;
    int max_items;
};
inline Buffers buffers_of(const BlockArgs &a) {
    const Layout l = layout_for(a.S, a.topk, a.H, a.MI, a.experts);
    unsigned char *ws = a.ws;
    Buffers b;
    b.perm = reinterpret_cast<int *>(ws + l.perm); b.pos = reinterpret_cast<int *>(ws + l.pos);
    b.offsets = reinterpret_cast<int *>(ws + l.offsets); b.num_items = reinterpret_cast<int *>(ws + l.num_items);
    b.items = reinterpret_cast<int4 *>(ws + l.items);
    b.xq = reinterpret_cast<int8_t *>(ws + l.xq); b.xq_g = reinterpret_cast<int8_t *>(ws + l.xq_g); b.xq_h = reinterpret_cast<int8_t *>(ws + l.xq_h);
    b.xs = reinterpret_cast<float *>(ws + l.xs); b.xs_g = reinterpret_cast<float *>(ws + l.xs_g); b.xs_h = reinterpret_cast<float *>(ws + l.xs_h);
    b.gu = reinterpret_cast<float *>(ws + l.gu); b.sout = reinterpret_cast<float *>(ws + l.sout);
    b.max_items = l.max_items;
    return b;
}

// Few slots on the grouped-GEMV path and a slot buffer that holds them: the tagged-slot row exchange.
inline bool tagged_rows(const BlockArgs &a, bool use_gemm) {
    return a.peers && !use_gemm && (size_t)a.S * a.topk * a.H <= LL_MAX_SLOTS;
}

// quantize, (sort, gather,) gate|up, activation + quantize, down; with peers: send this rank's rows on and publish
// (wait_limit > 0: and wait for every rank).
inline int launch_experts(const BlockArgs &a, const Buffers &b, bool use_gemm, long long wait_limit, cudaStream_t st) {
    const int nslots = a.S * a.topk, sms = sm_count();
    // Decode shape of benchmark configuration 5 (H <= 2048, MI = 768): the two grouped GEMVs produce their own activation
    // rows — quantize_x of the token's row in the prologue of gate|up, activation + quantize_x of the slot's gate|up row
    // in the prologue of down — so the block is three launches instead of five; same values in the same stage buffers.
    const bool fuse_rows = !use_gemm && a.H <= 64 * QBLK && a.H != 24 * QBLK && a.MI == 24 * QBLK && aligned(a.n2, 16) && aligned(a.dn_wq, 16) &&
                           aligned(b.xq_h, 16) && aligned(b.gu, 16) && (long)a.H * 24 < (1L << 30);
    int rc = W4A8_OK;
    if (!fuse_rows) rc = launch_quantize_x(a.n2, b.xq, b.xs, nullptr, a.H, a.S, st);
    if (rc != W4A8_OK) return rc;
    if (use_gemm) {
        moe_sort_kernel<<<1, 1024, 0, st>>>(a.idx, nslots, a.expert_base, a.experts, b.perm, b.pos, b.offsets, b.items, b.num_items);
        rc = launch_status("moe_sort");
        if (rc != W4A8_OK) return rc;
    }
    if (use_gemm) {
        const unsigned gg = (unsigned)(nslots < sms * 8 ? nslots : sms * 8);
        moe_gather_rows_kernel<<<gg, 128, 0, st>>>(b.xq, b.xs, b.perm, b.offsets + a.experts, a.topk, a.H, b.xq_g, b.xs_g);
        rc = launch_status("moe_gather_rows");
        if (rc != W4A8_OK) return rc;
        gemm::GroupList gl;
        gl.items = b.items; gl.num_items = b.num_items;
        rc = gemm::launch_tc_grouped(b.xq_g, b.xs_g, a.gu_wq, a.gu_sc, b.gu, nslots, 2 * a.MI, a.H, a.scale_dtype, a.experts, gl, b.max_items, st);
        if (rc != W4A8_OK) return rc;
        rc = launch_glu_quantize(b.gu, b.gu + a.MI, a.act, nullptr, b.xq_h, b.xs_h, nullptr, a.MI, nslots, st, 2L * a.MI);
        if (rc != W4A8_OK) return rc;
        rc = gemm::launch_tc_grouped(b.xq_h, b.xs_h, a.dn_wq, a.dn_sc, b.sout, nslots, a.H, a.MI, a.scale_dtype, a.experts, gl, b.max_items, st);
        if (rc != W4A8_OK) return rc;
    } else if (fuse_rows) {
        GroupedArgs f1, f2;
        f1.src_mode = 1; f1.src_f32 = a.n2; f1.xq_out = b.xq; f1.xs_out = b.xs;
        rc = launch_moe_gemv(b.xq, b.xs, a.gu_wq, a.gu_sc, a.idx, b.gu, nslots, a.topk, 0, 2 * a.MI, a.H, a.experts, a.scale_dtype, st, a.expert_base, a.world, &f1);
        if (rc != W4A8_OK) return rc;
        f2.src_mode = 2; f2.act = a.act; f2.src_f32 = b.gu; f2.xq_out = b.xq_h; f2.xs_out = b.xs_h;
        rc = launch_moe_gemv(b.xq_h, b.xs_h, a.dn_wq, a.dn_sc, a.idx, b.sout, nslots, a.topk, 1, a.H, a.MI, a.experts, a.scale_dtype, st, a.expert_base, a.world, &f2);
        if (rc != W4A8_OK) return rc;
    } else {
        rc = launch_moe_gemv(b.xq, b.xs, a.gu_wq, a.gu_sc, a.idx, b.gu, nslots, a.topk, 0, 2 * a.MI, a.H, a.experts, a.scale_dtype, st, a.expert_base, a.world);
        if (rc != W4A8_OK) return rc;
        rc = launch_glu_quantize(b.gu, b.gu + a.MI, a.act, nullptr, b.xq_h, b.xs_h, nullptr, a.MI, nslots, st, 2L * a.MI, true);
        if (rc != W4A8_OK) return rc;
        rc = launch_moe_gemv(b.xq_h, b.xs_h, a.dn_wq, a.dn_sc, a.idx, b.sout, nslots, a.topk, 1, a.H, a.MI, a.experts, a.scale_dtype, st, a.expert_base, a.world);
        if (rc != W4A8_OK) return rc;
    }
    if (a.peers && tagged_rows(a, use_gemm)) {
        const unsigned pg = (unsigned)(nslots < sms * 4 ? nslots : sms * 4);
        moe_push_rows_ll_kernel<<<pg, 256, 0, st>>>(a.peers, b.sout, a.idx, nslots, a.H, a.expert_base, a.experts, a.epoch);
        rc = launch_status("moe_push_rows_ll");
    } else if (a.peers) {
        const unsigned pg = (unsigned)(nslots < sms * 4 ? nslots : sms * 4);
        moe_push_rows_kernel<<<pg, 256, 0, st>>>(a.peers, reinterpret_cast<const float4 *>(b.sout), use_gemm ? 1 : 0, use_gemm ? b.perm : nullptr,
                                                  b.offsets + a.experts, a.H / 4, a.sout_off, a.epoch, wait_limit, a.idx, nslots, a.expert_base,
                                                  a.experts);
        rc = launch_status("moe_push_rows");
    }
    return rc;
}

inline int launch_block(const BlockArgs &a, cudaStream_t st) {
    const int nslots = a.S * a.topk, sms = sm_count();
    const Buffers b = buffers_of(a);
    const bool use_gemm = a.kernel == 2 || (a.kernel == 0 && nslots > GEMV_MAX_SLOTS);
    int rc = W4A8_OK;
    const bool tagged = tagged_rows(a, use_gemm);
    if (a.peers && a.phase == 2) {
        if (!tagged) {
            allgather_wait_kernel<<<1, 32, 0, st>>>(a.peers, a.epoch, a.wait_limit);
            rc = launch_status("allgather_wait");
        }
    } else {
        rc = launch_experts(a, b, use_gemm, a.phase == 1 ? 0 : a.wait_limit, st);
    }
    if (rc != W4A8_OK || (a.peers && a.phase == 1)) return rc;
    if (tagged) {
        // local slots from this rank's own down outputs, the others from the slot buffer the other ranks fill
        const long tot = (long)a.S * a.H;
        const long wantc = (tot + 255) / 256;
        const unsigned cgl = (unsigned)(wantc < (long)sms * 8 ? (wantc > 0 ? wantc : 1) : (long)sms * 8);
        moe_combine_ll_kernel<<<cgl, 256, 0, st>>>(a.peers, b.sout, a.idx, a.dw, a.out, a.H, a.topk, tot, a.expert_base, a.experts, a.epoch,
                                                    a.wait_limit);
        return launch_status("moe_combine_ll");
    }
    // one GPU: the down outputs as computed (sorted rows through pos, or slot order); expert shard: the slot-ordered
    // buffer of this rank's arena, complete once every rank's flag has arrived
    const float4 *src = a.peers ? reinterpret_cast<const float4 *>(a.arena_base + a.sout_off) : reinterpret_cast<const float4 *>(b.sout);
    const int *pos = (!a.peers && use_gemm) ? b.pos : nullptr;
    const long total = (long)a.S * (a.H / 4);
    const long want = (total + 255) / 256;
    const unsigned cg = (unsigned)(want < (long)sms * 8 ? (want > 0 ? want : 1) : (long)sms * 8);
    // the grouped GEMVs before it are launched for programmatic dependent launch; so is the combine (it waits first)
    const cudaError_t le = launch_pdl(moe_combine_kernel, dim3(cg), dim3(256), 0, st, src, pos, a.dw, reinterpret_cast<float4 *>(a.out), a.H / 4,
                                      a.topk, total);
    if (le != cudaSuccess) return cuda_fail(le, "moe_combine launch");
    return launch_status("moe_combine");
}

}  // namespace moe
}  // namespace w4a8
