// W4A8 decode GEMV for 1..16 activation rows on the 5th-generation tensor cores, weights on the M side of the MMA.
//   Y[s,o] = sum_b ((float)D[s,o,b] * xs[s,b]) * sw[o,b],   D[s,o,b] = sum_{k in group b} xq[s,k] * (Wq[o,k] - 8)
// Same product as the reference's kernels/gemv_w4a8.cuh:24-151 and gemm_batch.cuh:177-231; fp32 evaluation in the MMQ
// order of kernels/gemm_mmq.cuh:104-105 (t = (float)D*xs; acc = fma(t, sw, acc), groups ascending), so a row's bits
// are those of w4a8_gemm and do not depend on S: decoded alone or in a batch, a row is the same (the batch == single
// rule of tools/probe_mlp_vs_sb.cu:1-2 and models/qwen35_batch.cu:262-275).
//
// Why tensor cores for a matrix-vector product.  The 4-way byte dot product is not a single instruction on sm_100a: the
// CUDA-core kernels (csrc/gemv_w4a8.cuh, gemv_w4a8_bulk.cuh) execute 60 to 90 warp instructions per 32 (row, group)
// pairs where their source has 26, and the decode GEMV is bound by issue slots before it is bound by HBM (a copy-only
// pipeline streams the same matrix a quarter faster).  Here one tcgen05.mma (kind::i8, M = 128 weight rows, N = 16
// activation rows, K = 32 = one group) produces the exact int32 dots of 128 rows x 16 activation rows; what is left
// for the CUDA cores is the int4 -> int8 expansion of the weights (per 8 packed bytes one load, six logic operations
// and one store) and three fp32 operations per (row, group, s).
//
// One CTA per SM owns a contiguous range of output rows and walks it in tiles of at most 128 rows; K goes in K-tiles
// of 256 elements (8 groups).  Roles:
//   warps 0, 2  TMA producers (one thread each): packed weights [rows x 128 B] per K-tile; weight scales [rows x 128 B] per
//               32 groups (fp16: 64); each behind its own mbarrier ring.  Weights are never written by a kernel of the stream,
//               so they do not wait for the previous kernel (programmatic dependent launch).
//   warps 8-11  MMA issuers (one thread each): per group one tcgen05.mma into a 16-column slice of a TMEM buffer, four groups
//               per buffer and commit; tcgen05.commit also releases the operand stages.  Several issuers because one thread
//               gets out one MMA per ~250 cycles however small it is.
//   warp 1      activation operand: waits for the previous kernel, stages xs (times the exact 1/16 that undoes the 16x of
//               the expansion) in shared memory and, per K-tile, writes the 16 x 256 bytes of activations into the
//               swizzled K-major B operand (rows past S are zero).
//   warps 16-19 expand int4 -> int8 (as 16*(w-8), unpack8_x16) from the packed stage into the swizzled K-major A operand.
//               The expansion keeps the even / odd order unpack8_x16 produces; the activation operand is permuted the
//               same way, and a permutation of k inside one MMA does not change its sum.
//   warps 4-7   epilogue: lane = output row.  tcgen05.ld of the group dots, then for every activation row
//               t = (float)d * xs, acc = fma(t, sw, acc) with the accumulators in registers; Y is stored per tile.
// Every mbarrier wait is bounded (device error word on expiry, TMEM is freed on every path).  No cluster multicast.
//
// Preconditions (else the caller uses another kernel): S <= 16, K % 128 == 0 (K % 256 == 0 with fp16 scales), xq, Wq and
// sw 16-byte aligned.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "peer_allgather.cuh"
#include "gemv_w4a8.cuh"
#include "tmap_cache.cuh"

namespace w4a8 {
namespace gemv_tc {

constexpr int TM = 128;            // weight rows per tile (MMA M = TMEM lanes)
constexpr int TN = 16;             // MMA N: activation rows, padded
constexpr int KT = 256;            // K elements per K-tile
constexpr int GPK = KT / QBLK;     // groups per K-tile (8)
#ifndef W4A8_TC_GPB
#define W4A8_TC_GPB 4
#endif
#ifndef W4A8_TC_XW
#define W4A8_TC_XW 4
#endif
constexpr int GPB = W4A8_TC_GPB;   // groups per TMEM buffer (one commit): 4 (or 2)
constexpr int BPK = GPK / GPB;     // TMEM buffers per K-tile (the later ones are empty in a last K-tile of 4 groups)
constexpr int TB = 16 / GPB;       // TMEM buffers in flight: TB * GPB * TN = 256 columns
constexpr int EPB = 4 / GPB;       // buffers the epilogue takes at a time (always four groups)
// One thread issues a tcgen05.mma about every 250 cycles whatever its N (measured: 252 cycles at N = 16 and 245 at
// N = 256, back to back, one thread), but several issuing threads each keep that rate side by side, so the 160 small
// MMAs of a 128-row tile go out through NI threads of different warps: issuer i owns the TMEM buffers i, i + NI, ...
// With NI = TB and S8 = 2 every issuer always meets the same TMEM buffer and the same operand stage, use after use,
// so none of its parity waits can be more than one phase ahead.
constexpr int NI = TB;
constexpr int XW = W4A8_TC_XW;     // expansion warps (4 or 8)
constexpr int MAX_SP = 6;          // packed-weight stages: as many as fit (runtime), at most this
constexpr int S8 = 2;              // expanded-weight stages
constexpr int SC = 2;              // scale stages
constexpr int SBA = 4;             // activation-operand stages
constexpr int RD = 8;              // raw-activation ring: K-tiles in flight (cp.async)
constexpr int BP_STAGE = TM * KT / 2;      // 16 KB
constexpr int A8_STAGE = TM * KT;          // 32 KB: two [128 x 128 B] swizzle atoms
constexpr int SC_STAGE = TM * 128;         // 16 KB
constexpr int B_STAGE = TN * KT;           // 4 KB: two [16 x 128 B] atoms
constexpr int OFF_A8 = 0;
constexpr int OFF_SC = OFF_A8 + S8 * A8_STAGE;
constexpr int OFF_B = OFF_SC + SC * SC_STAGE;
constexpr int OFF_BAR = OFF_B + SBA * B_STAGE;
constexpr int NUM_BARS = 2 * (MAX_SP + S8 + SC + SBA + TB) + 1;
constexpr int OFF_TMEM = OFF_BAR + NUM_BARS * 8;
constexpr int OFF_BP = (OFF_TMEM + 16 + 127) & ~127;         // packed stages [sp][16 KB], then raw activations, then xs16
constexpr int THREADS = (16 + XW) * 32;   // warps: 0 TMA weights, 1 activations, 2 TMA scales, 4-7 epilogue, 8.. MMA issuers, 16.. expansion
constexpr int TMEM_COLS = TB * GPB * TN;

enum : unsigned { ERR_PRODUCER = 0x610, ERR_MMA = 0x620, ERR_ACT = 0x630, ERR_EXPAND = 0x640, ERR_EPILOGUE = 0x650 };

struct Ring {
    int stage = 0;
    uint32_t phase = 0;
    const int depth;
    __device__ explicit Ring(int d) : depth(d) {}
    __device__ __forceinline__ void advance() { if (++stage == depth) { stage = 0; phase ^= 1u; } }
};

// Rows of tile t of a CTA that owns rows [r0, r1) in `ntile` tiles.
__device__ __forceinline__ void tile_range(int r0, int r1, int ntile, int t, int &a, int &b) {
    const long rows = r1 - r0;
    a = r0 + (int)((rows * t) / ntile);
    b = r0 + (int)((rows * (t + 1)) / ntile);
}

__device__ __forceinline__ void load_sw4(const unsigned char *p, float (&s)[4], float) {
    const float4 v = *reinterpret_cast<const float4 *>(p);
    s[0] = v.x; s[1] = v.y; s[2] = v.z; s[3] = v.w;
}
__device__ __forceinline__ void load_sw4(const unsigned char *p, float (&s)[4], __half) {
    const uint2 v = *reinterpret_cast<const uint2 *>(p);
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&v.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&v.y));
    s[0] = a.x; s[1] = a.y; s[2] = b.x; s[3] = b.y;
}

// NC = columns of the accumulator the epilogue reads = S rounded up to 1, 2, 4, 8 or 16.
template <int NC, typename ST, bool PEER>
__global__ void __launch_bounds__(THREADS, 1) gemv_w4a8_tc_kernel(
    const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmS, const int8_t *__restrict__ xq,
    const float *__restrict__ xs, float *__restrict__ Y, int IN, int OUT, int S, int ntile, int box_rows, int row_base,
    int sp, OutArgs oa) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw = ptx::smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char *base_ptr = smem_dyn + (base - raw);
    const uint32_t bar0 = base + OFF_BAR;
    auto BAR = [&](int idx) { return bar0 + 8u * idx; };
    constexpr int BP_FULL = 0, BP_EMPTY = BP_FULL + MAX_SP, A8_FULL = BP_EMPTY + MAX_SP, A8_EMPTY = A8_FULL + S8,
                  SC_FULL = A8_EMPTY + S8, SC_EMPTY = SC_FULL + SC, B_FULL = SC_EMPTY + SC, B_EMPTY = B_FULL + SBA,
                  TM_FULL = B_EMPTY + SBA, TM_EMPTY = TM_FULL + TB, XS_FULL = TM_EMPTY + TB;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + OFF_TMEM);
    unsigned char *rawx = base_ptr + OFF_BP + sp * BP_STAGE;     // raw activations [RD][S][256 B]
    float *xs16 = reinterpret_cast<float *>(rawx + (size_t)RD * S * KT);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = IN / QBLK;
    const int nkt = (nb + GPK - 1) / GPK;
    constexpr int SGB = 128 / (int)sizeof(ST);           // groups per scale box row (32 fp32, 64 fp16)
    constexpr int KTS = SGB / GPK;                       // K-tiles per scale box (4, 8)
    const int r0 = (int)(((long)OUT * blockIdx.x) / gridDim.x), r1 = (int)(((long)OUT * (blockIdx.x + 1)) / gridDim.x);
    const int nt = r1 > r0 ? ntile : 0;

    if (tid == 0) {
        for (int i = 0; i < sp; i++) { ptx::mbar_init(BAR(BP_FULL + i), 1); ptx::mbar_init(BAR(BP_EMPTY + i), XW); }
        for (int i = 0; i < S8; i++) { ptx::mbar_init(BAR(A8_FULL + i), XW); ptx::mbar_init(BAR(A8_EMPTY + i), BPK); }
        for (int i = 0; i < SC; i++) { ptx::mbar_init(BAR(SC_FULL + i), 1); ptx::mbar_init(BAR(SC_EMPTY + i), 4); }
        for (int i = 0; i < SBA; i++) { ptx::mbar_init(BAR(B_FULL + i), 1); ptx::mbar_init(BAR(B_EMPTY + i), BPK); }
        for (int i = 0; i < TB; i++) { ptx::mbar_init(BAR(TM_FULL + i), 1); ptx::mbar_init(BAR(TM_EMPTY + i), 4); }
        ptx::mbar_init(BAR(XS_FULL), 1);
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(&tmW);
        ptx::tma_prefetch_desc(&tmS);
    }
    if (warp == 3) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();

    if (warp == 0) {
        // ---------------- TMA producer, packed weights: one box per K-tile ----------------
        if (lane == 0) {
            Ring rp(sp);
            bool ok = true;
            for (int t = 0; t < nt && ok; t++) {
                int ta, tb;
                tile_range(r0, r1, ntile, t, ta, tb);
                for (int kt = 0; kt < nkt && ok; kt++) {
                    if (!ptx::mbar_wait(BAR(BP_EMPTY + rp.stage), rp.phase ^ 1u)) { dev_set_error(ERR_PRODUCER | 2); ok = false; break; }
                    ptx::mbar_arrive_expect_tx(BAR(BP_FULL + rp.stage), (uint32_t)box_rows * 128u);
                    ptx::tma_load_2d(base + OFF_BP + rp.stage * BP_STAGE, &tmW, kt * 128, row_base + ta, BAR(BP_FULL + rp.stage));
                    rp.advance();
                }
            }
            if (!ok) {  // give copies already in flight time to land before the CTA's shared memory goes away
                const long long t0 = clock64();
                while (clock64() - t0 < (1ll << 21)) { }
            }
        }
    } else if (warp == 2) {
        // ---------------- TMA producer, weight scales: one box per KTS K-tiles.  A thread of its own: the scale ring is
        // released by the epilogue, K-tiles later than the packed stages are, and a producer that waited for it could not
        // run ahead with the weights.
        if (lane == 0) {
            Ring rc(SC);
            bool ok = true;
            for (int t = 0; t < nt && ok; t++) {
                int ta, tb;
                tile_range(r0, r1, ntile, t, ta, tb);
                for (int kt = 0; kt < nkt && ok; kt += KTS) {
                    if (!ptx::mbar_wait(BAR(SC_EMPTY + rc.stage), rc.phase ^ 1u)) { dev_set_error(ERR_PRODUCER | 1); ok = false; break; }
                    ptx::mbar_arrive_expect_tx(BAR(SC_FULL + rc.stage), (uint32_t)box_rows * 128u);
                    ptx::tma_load_2d(base + OFF_SC + rc.stage * SC_STAGE, &tmS, (kt / KTS) * 128, row_base + ta, BAR(SC_FULL + rc.stage));
                    rc.advance();
                }
            }
            if (!ok) {
                const long long t0 = clock64();
                while (clock64() - t0 < (1ll << 21)) { }
            }
        }
    } else if (warp >= 8 && warp < 8 + NI) {
        // ---------------- MMA issuers: issuer `me` takes the TMEM buffers n = me, me + NI, ... ----------------
        const int me = warp - 8;
        if (lane == 0) {
            const uint32_t idesc = ptx::umma_idesc_s8(TM, TN);
            bool ok = true;
            const int nitem = nt * nkt;                              // items = (tile, K-tile) pairs; BPK buffers each
            for (int n = me; n < nitem * BPK && ok; n += NI) {
                const int item = n / BPK, gb = n % BPK, kt = item % nkt;
                const int s8 = item % S8, sb = item % SBA, stage = n % TB;
                if (!ptx::mbar_wait(BAR(A8_FULL + s8), (uint32_t)(item / S8) & 1u)) { dev_set_error(ERR_MMA | 1); ok = false; break; }
                if (!ptx::mbar_wait(BAR(B_FULL + sb), (uint32_t)(item / SBA) & 1u)) { dev_set_error(ERR_MMA | 2); ok = false; break; }
                if (!ptx::mbar_wait(BAR(TM_EMPTY + stage), ((uint32_t)(n / TB) & 1u) ^ 1u)) { dev_set_error(ERR_MMA | 3); ok = false; break; }
                ptx::tc_fence_after_sync();
                const int ng = min(GPK, nb - kt * GPK);              // a multiple of 4 (nb % 4 == 0)
                if (gb * GPB < ng) {
#pragma unroll
                    for (int q = 0; q < GPB; q++) {
                        const int g = gb * GPB + q;                  // group inside the K-tile: atom g / 4, bytes [32*(g%4), +32) of the row
                        const uint64_t adesc = ptx::umma_desc_k_sw128(base + OFF_A8 + s8 * A8_STAGE + (g >> 2) * (TM * 128)) + (uint64_t)((g & 3) * 2);
                        const uint64_t bdesc = ptx::umma_desc_k_sw128(base + OFF_B + sb * B_STAGE + (g >> 2) * (TN * 128)) + (uint64_t)((g & 3) * 2);
                        ptx::umma_i8(tmem_base + (uint32_t)(stage * GPB * TN + q * TN), adesc, bdesc, idesc, 0u);
                    }
                }
                // an empty buffer (second half of a K-tile of 4 groups) still completes its phases: the counts stay uniform
                ptx::umma_commit(BAR(TM_FULL + stage));
                ptx::umma_commit(BAR(A8_EMPTY + s8));
                ptx::umma_commit(BAR(B_EMPTY + sb));
            }
        }
    } else if (warp == 1) {
        // ---------------- activation operand (depends on the previous kernel) ----------------
        // The raw bytes of a K-tile (S rows x 256 B, L2-resident) are fetched RD K-tiles ahead with cp.async: a
        // synchronous load per K-tile would put an L2 round trip on the path of every K-tile of the CTA.
        pdl_wait();
        for (int i = lane; i < S * nb; i += 32) xs16[i] = xs[i] * 0.0625f;   // exact 1/16
        // rows past S of every stage stay zero for the whole kernel
        for (int i = lane; i < SBA * B_STAGE / 16; i += 32) reinterpret_cast<uint4 *>(base_ptr + OFF_B)[i] = make_uint4(0, 0, 0, 0);
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(BAR(XS_FULL));
        const int total = nt * nkt;                                  // items = (tile, K-tile) pairs
        const uint32_t raw_u32 = ptx::smem_u32(rawx);
        // task = (activation row m, 16-byte chunk c of the K-tile); a lane copies and later reads back its own tasks only
        auto fetch = [&](int item) {
            if (item < total) {
                const int kt = item % nkt;
                for (int task = lane; task < S * 16; task += 32) {
                    const int m = task >> 4, c = task & 15;
                    const int k0 = kt * KT + c * 16;
                    if (k0 < IN) {
                        const uint32_t dsta = raw_u32 + (uint32_t)((item % RD) * S * KT + task * 16);
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dsta), "l"(xq + (size_t)m * IN + k0) : "memory");
                    }
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");     // one group per item, empty or not: the count stays uniform
        };
        for (int item = 0; item < RD - 1; item++) fetch(item);
        Ring rb(SBA);
        bool ok = true;
        for (int item = 0; item < total && ok; item++) {
            const int kt = item % nkt;
            fetch(item + RD - 1);
            asm volatile("cp.async.wait_group %0;" ::"n"(RD - 1) : "memory");   // item `item` has landed
            if (!ptx::mbar_wait_warp(BAR(B_EMPTY + rb.stage), rb.phase ^ 1u)) { dev_set_error(ERR_ACT | 1); ok = false; break; }
            unsigned char *dst = base_ptr + OFF_B + rb.stage * B_STAGE;
            const unsigned char *src = rawx + (size_t)(item % RD) * S * KT;
            for (int task = lane; task < S * 16; task += 32) {       // 16 elements -> [e o e o] in unpack8_x16 order
                const int m = task >> 4, c = task & 15;
                const int k0 = kt * KT + c * 16;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (k0 < IN) v = *reinterpret_cast<const uint4 *>(src + task * 16);
                uint4 o;
                split_even_odd(v.x, v.y, o.x, o.y);
                split_even_odd(v.z, v.w, o.z, o.w);
                *reinterpret_cast<uint4 *>(dst + (c >> 3) * (TN * 128) + m * 128 + (((c & 7) ^ (m & 7)) << 4)) = o;
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(BAR(B_FULL + rb.stage));
            rb.advance();
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else if (warp >= 16) {
        // ---------------- int4 -> int8 expansion into the swizzled A operand ----------------
        const int dt = tid - 16 * 32;                                // 0 .. XW*32-1
        Ring rp(sp), r8(S8);
        bool ok = true;
        for (int t = 0; t < nt && ok; t++) {
            for (int kt = 0; kt < nkt && ok; kt++) {
                bool w = ptx::mbar_wait_warp(BAR(BP_FULL + rp.stage), rp.phase);
                w = w && ptx::mbar_wait_warp(BAR(A8_EMPTY + r8.stage), r8.phase ^ 1u);
                if (!w) { dev_set_error(ERR_EXPAND | 1); ok = false; break; }
                const unsigned char *src = base_ptr + OFF_BP + rp.stage * BP_STAGE;
                unsigned char *dst = base_ptr + OFF_A8 + r8.stage * A8_STAGE;
                // task j = (row n, 8 packed bytes c = 16 weights = one 16-byte chunk of the operand); all loads of a half
                // first, then expansion and stores (the compiler cannot tell that the two stages do not overlap)
                constexpr int NT = (TM * 16) / (XW * 32);            // 8 tasks per thread
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    uint2 pk[NT / 2];
#pragma unroll
                    for (int i = 0; i < NT / 2; i++) {
                        const int j = dt + (h * (NT / 2) + i) * (XW * 32);
                        pk[i] = *reinterpret_cast<const uint2 *>(src + (j >> 4) * 128 + (j & 15) * 8);
                    }
#pragma unroll
                    for (int i = 0; i < NT / 2; i++) {
                        const int j = dt + (h * (NT / 2) + i) * (XW * 32);
                        const int n = j >> 4, c = j & 15;
                        uint4 o;
                        unpack8_x16(pk[i].x, o.x, o.y);
                        unpack8_x16(pk[i].y, o.z, o.w);
                        *reinterpret_cast<uint4 *>(dst + (c >> 3) * (TM * 128) + n * 128 + (((c & 7) ^ (n & 7)) << 4)) = o;
                    }
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) { ptx::mbar_arrive(BAR(A8_FULL + r8.stage)); ptx::mbar_arrive(BAR(BP_EMPTY + rp.stage)); }
                rp.advance();
                r8.advance();
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ---------------- epilogue: lane = output row ----------------
        const int quad = warp & 3;                                   // TMEM lanes [32*quad, 32*quad+32)
        const int rloc = quad * 32 + lane;                           // row inside the tile
        Ring rc(SC);
        int nbuf = 0;                                                // running TMEM buffer number of the CTA
        bool ok = ptx::mbar_wait_warp(BAR(XS_FULL), 0u);
        if (!ok) dev_set_error(ERR_EPILOGUE | 4);
        for (int t = 0; t < nt && ok; t++) {
            int ta, tb;
            tile_range(r0, r1, ntile, t, ta, tb);
            float acc[NC];
#pragma unroll
            for (int m = 0; m < NC; m++) acc[m] = 0.f;
            const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16);
            for (int kt = 0; kt < nkt && ok; kt++) {
                const int ng = min(GPK, nb - kt * GPK);
                for (int gb = 0; gb < BPK && ok; gb += EPB) {        // EPB buffers = four groups at a time
                    const int b0 = kt * GPK + gb * GPB;              // first group of these buffers
                    const bool live = gb * GPB < ng;                 // else: the empty second half of a short last K-tile
                    const int stage = nbuf % TB;                     // the buffers are stage .. stage + EPB - 1
                    const uint32_t par = (uint32_t)(nbuf / TB) & 1u;
                    nbuf += EPB;
                    if (live && b0 % SGB == 0) {
                        if (!ptx::mbar_wait_warp(BAR(SC_FULL + rc.stage), rc.phase)) { dev_set_error(ERR_EPILOGUE | 1); ok = false; break; }
                    }
                    bool tw = ptx::mbar_wait_warp(BAR(TM_FULL + stage), par);
                    if (EPB == 2) tw = tw && ptx::mbar_wait_warp(BAR(TM_FULL + stage + EPB - 1), par);
                    if (!tw) { dev_set_error(ERR_EPILOGUE | 2); ok = false; break; }
                    ptx::tc_fence_after_sync();
                    if (!live) {
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) { ptx::mbar_arrive(BAR(TM_EMPTY + stage)); if (EPB == 2) ptx::mbar_arrive(BAR(TM_EMPTY + stage + EPB - 1)); }
                        continue;
                    }
                    uint32_t d[4][NC];                               // the pair's columns are contiguous: 4 groups x 16 columns
#pragma unroll
                    for (int q = 0; q < 4; q++) ptx::tmem_ld(tlane + (uint32_t)(stage * GPB * TN + q * TN), d[q]);
                    // this row's four scales of the groups b0 .. b0+3: one 16-byte (fp16: 8-byte) load from the swizzled box
                    float sw4[4];
                    {
                        const int gi = b0 % SGB;                      // group inside the scale box
                        const int byte = gi * (int)sizeof(ST);        // byte inside the row's 128
                        const unsigned char *srow = base_ptr + OFF_SC + rc.stage * SC_STAGE + rloc * 128;
                        load_sw4(srow + ((((byte >> 4) ^ (rloc & 7)) << 4) | (byte & 15)), sw4, ST());
                    }
                    ptx::tmem_ld_wait();
                    ptx::tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) { ptx::mbar_arrive(BAR(TM_EMPTY + stage)); if (EPB == 2) ptx::mbar_arrive(BAR(TM_EMPTY + stage + EPB - 1)); }
#pragma unroll
                    for (int q = 0; q < 4; q++) {
#pragma unroll
                        for (int m = 0; m < NC; m++) {
                            if (m < S) {
                                const float tq = (float)(int)d[q][m] * xs16[m * nb + b0 + q];   // = (float)D * xs, rounded once
                                acc[m] = fmaf(tq, sw4[q], acc[m]);
                            }
                        }
                    }
                    if ((b0 + 4) % SGB == 0 || b0 + 4 >= nb) {        // done with this scale box
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(BAR(SC_EMPTY + rc.stage));
                        rc.advance();
                    }
                }
            }
            if (!ok) break;
            const int row = ta + rloc;
            if (row < tb) {
#pragma unroll
                for (int m = 0; m < NC; m++)
                    if (m < S) store_out<PEER>(Y, oa, OUT, m, row, acc[m]);
            }
        }
    }

    publish_out<PEER>(oa, warp >= 4 && warp < 8);
    // ---------------- teardown ----------------
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 3) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side --------------------------------------------------------------------------------------------------
inline int packed_stages(int S, int IN);
inline bool supported(const void *xq, const void *Wq, const void *sw, int IN, int S, int scale_dtype) {
    const int need = scale_dtype == 1 ? 256 : 128;
    return IN > 0 && IN % need == 0 && S >= 1 && S <= TN && aligned(xq, 16) && aligned(Wq, 16) && aligned(sw, 16) &&
           packed_stages(S, IN) >= 2;
}

// Packed-weight stages: as many as fit beside the fixed buffers, the raw-activation ring and xs16 (2 at least).
inline int packed_stages(int S, int IN) {
    const long fixed = OFF_BP + (long)RD * S * KT + (long)S * (IN / QBLK) * 4 + 1024;
    long sp = ((long)227 * 1024 - fixed) / BP_STAGE;
    return (int)(sp > MAX_SP ? MAX_SP : sp);
}
inline size_t smem_bytes(int S, int IN, int sp) {
    return (size_t)OFF_BP + (size_t)sp * BP_STAGE + (size_t)RD * S * KT + (size_t)S * (IN / QBLK) * 4 + 1024;
}

template <int NC, typename ST, bool PEER>
inline int launch_k(const CUtensorMap &tmW, const CUtensorMap &tmS, const int8_t *xq, const float *xs, float *Y, int IN, int OUT,
                    int S, unsigned grid, int ntile, int box_rows, int row_base, cudaStream_t st, const OutArgs &oa) {
    auto kern = gemv_w4a8_tc_kernel<NC, ST, PEER>;
    const int sp = packed_stages(S, IN);
    const size_t smem = smem_bytes(S, IN, sp);
    if (sp < 2 || smem > 227 * 1024) return fail(W4A8_ERR_UNSUPPORTED, "gemv_tc: %zu bytes of shared memory needed", smem);
    static PerDevice<size_t> configured;                 // grow-only; the opt-in is a per-device function attribute
    size_t &c = configured.get();
    if (smem > c) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return cuda_fail(e, "gemv_tc smem opt-in");
        c = smem;
    }
    cudaError_t le = launch_pdl(kern, dim3(grid), dim3(THREADS), smem, st, tmW, tmS, xq, xs, Y, IN, OUT, S, ntile, box_rows, row_base, sp, oa);
    if (le != cudaSuccess) return cuda_fail(le, "gemv_w4a8_tc launch");
    return launch_status("gemv_w4a8_tc");
}

template <typename ST, bool PEER>
inline int launch_t(const CUtensorMap &tmW, const CUtensorMap &tmS, const int8_t *xq, const float *xs, float *Y, int IN, int OUT,
                    int S, unsigned grid, int ntile, int box_rows, int row_base, cudaStream_t st, const OutArgs &oa) {
    if (S <= 1) return launch_k<1, ST, PEER>(tmW, tmS, xq, xs, Y, IN, OUT, S, grid, ntile, box_rows, row_base, st, oa);
    if (S <= 2) return launch_k<2, ST, PEER>(tmW, tmS, xq, xs, Y, IN, OUT, S, grid, ntile, box_rows, row_base, st, oa);
    if (S <= 4) return launch_k<4, ST, PEER>(tmW, tmS, xq, xs, Y, IN, OUT, S, grid, ntile, box_rows, row_base, st, oa);
    if (S <= 8) return launch_k<8, ST, PEER>(tmW, tmS, xq, xs, Y, IN, OUT, S, grid, ntile, box_rows, row_base, st, oa);
    return launch_k<16, ST, PEER>(tmW, tmS, xq, xs, Y, IN, OUT, S, grid, ntile, box_rows, row_base, st, oa);
}

// rows_total = rows of the whole tensor behind Wq / sw (OUT for a dense matrix); row_base = first row of this matrix in it.
inline int launch(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int IN, int OUT, int S,
                  int scale_dtype, cudaStream_t st, const OutArgs &oa, long rows_total = 0, int row_base = 0) {
    if (S == 0 || OUT == 0) return W4A8_OK;
    if (rows_total <= 0) rows_total = OUT;
    const int nsm = sm_count();
    long grid = (OUT + 7) / 8;                           // fewer than 8 rows per CTA only adds launch overhead
    if (grid > nsm) grid = nsm;
    const int rmax = (int)((OUT + grid - 1) / grid);     // rows of the largest CTA
    const int ntile = (rmax + TM - 1) / TM;
    const int box_rows = (rmax + ntile - 1) / ntile;     // rows of the largest tile: every tile is fetched with this box
    const size_t ssz = scale_dtype == 1 ? 2 : 4;
    CUtensorMap mW, mS;
    int rc = tmap_cached(&mW, Wq, (uint64_t)IN / 2, (uint64_t)rows_total, 128, (uint32_t)box_rows, CU_TENSOR_MAP_SWIZZLE_NONE,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != W4A8_OK) return rc;
    rc = tmap_cached(&mS, sw, (uint64_t)(IN / QBLK) * ssz, (uint64_t)rows_total, 128, (uint32_t)box_rows, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
    if (rc != W4A8_OK) return rc;
    if (scale_dtype == 1) {
        if (oa.peers) return launch_t<__half, true>(mW, mS, xq, xs, Y, IN, OUT, S, (unsigned)grid, ntile, box_rows, row_base, st, oa);
        return launch_t<__half, false>(mW, mS, xq, xs, Y, IN, OUT, S, (unsigned)grid, ntile, box_rows, row_base, st, oa);
    }
    if (oa.peers) return launch_t<float, true>(mW, mS, xq, xs, Y, IN, OUT, S, (unsigned)grid, ntile, box_rows, row_base, st, oa);
    return launch_t<float, false>(mW, mS, xq, xs, Y, IN, OUT, S, (unsigned)grid, ntile, box_rows, row_base, st, oa);
}

}  // namespace gemv_tc
}  // namespace w4a8
