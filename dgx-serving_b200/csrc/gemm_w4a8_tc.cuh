// W4A8 prefill / verify GEMM for sm_100a on the 5th-generation tensor cores.
//   Y[m,n] = sum_b ((float)D[m,n,b] * xs[m,b]) * sw[n,b],   D[m,n,b] = sum_{k in group b} X[m,k]*(Wq[n,k]-8)
// Semantics and fp32 evaluation order of the reference's kernels/gemm_mmq.cuh:38-120 (t = (float)c*xs,
// acc = fma(t, sw, acc), groups ascending, :104-105), shared by gemm_mma.cuh, gemm_mmq_tmpl.cuh,
// gemm_mmq_raster.cuh and gemm_mmq_ms.cuh.  Because both operands carry a scale per 32-element group,
// the tensor core can only produce ONE group's int32 dot per MMA (K = 32); the scaling and the sum over
// groups run on the CUDA cores, and that epilogue — three lane-operations per (m,n,group) — bounds the
// kernel, not the MMA rate.
//
// Persistent kernel, one CTA per SM, 128x128 output tile per step, warp-specialised:
//   warp 0      TMA producer: int8 activations [128 x 128 B] (128-byte swizzle) and packed int4 weights
//               [128 x 64 B] per K-tile of 128 elements, each behind its own mbarrier ring
//   warp 1      MMA issuer: one tcgen05.mma kind::i8 (128x128x32) per group into one of four 128-column
//               accumulator buffers in tensor memory; tcgen05.commit signals operand release / result ready
//   warps 2-3   expand int4 -> int8 (as 16*(w-8), see unpack8_x16) from the packed stage into the swizzled
//               K-major operand stage the MMA reads (generic-proxy writes + fence.proxy.async), and stage
//               both scale slices of the K-tile in shared memory: weight scales transposed to [group][n] and
//               pre-multiplied by the exact 1/16, activation scales transposed to [group][m]
//   warps 4-19  epilogue: tcgen05.ld the int32 group dots (lane = row, 32 columns per warp, loaded as two
//               16-column chunks so that one chunk's load is in flight while the other is processed), convert,
//               scale and accumulate in registers; store the fp32 tile at the end of the K loop.  The loop
//               touches no global memory.  Sixteen warps rather than eight because each warp's instruction
//               stream is a chain of waits (tensor-memory load, barrier, conversion pipe): four epilogue
//               warps per scheduler overlap them better than two (1253 -> 1214 us at M = 2048).
// Ragged M, N and a last partial K-tile are handled by TMA zero fill plus guards on scales and stores.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "peer_allgather.cuh"
#include "tmap_cache.cuh"

namespace w4a8 {
namespace gemm {

constexpr int BM = 128, BN = 128, KT = 128;
static_assert(BM == BN, "the grouped (transposed) instantiation exchanges the operands' roles");
constexpr int GPK = KT / QBLK;  // groups (MMAs) per K-tile = 4
#ifndef W4A8_GEMM_SA
#define W4A8_GEMM_SA 4
#endif
#ifndef W4A8_GEMM_SB
#define W4A8_GEMM_SB 4
#endif
constexpr int SA = W4A8_GEMM_SA;  // activation stages
constexpr int SB = W4A8_GEMM_SB;  // packed-weight stages
constexpr int S8 = 3;           // expanded-weight stages
constexpr int SS = 4;           // weight-scale stages
constexpr int TB = 4;           // TMEM accumulator buffers (TB * BN = 512 columns = all of tensor memory)
constexpr int A_STAGE = BM * KT;       // 16 KB
constexpr int BP_STAGE = BN * KT / 2;  // 8 KB
constexpr int B8_STAGE = BN * KT;      // 16 KB
constexpr int SW_STAGE = GPK * (BN + BM) * 4; // 4 KB: weight scales [group][n], then activation scales [group][m]
#ifndef W4A8_DEQ_WARPS
#define W4A8_DEQ_WARPS 2
#endif
#ifndef W4A8_EPI_UNROLL
#define W4A8_EPI_UNROLL 4
#endif
#ifndef W4A8_EPI_WARPS
#define W4A8_EPI_WARPS 16
#endif
constexpr int DEQ_WARPS = W4A8_DEQ_WARPS, EPI_WARPS = W4A8_EPI_WARPS;
constexpr int EPI_UNROLL = W4A8_EPI_UNROLL;
constexpr int EPI_COLS = BN / (EPI_WARPS / 4);  // accumulator columns per epilogue warp (32)
constexpr int EPI_CH = EPI_COLS / 2;           // columns per tcgen05.ld chunk (16)
constexpr int THREADS = (2 + DEQ_WARPS + EPI_WARPS) * 32;  // 640: up to 96 registers per thread
constexpr int OFF_A = 0;
constexpr int OFF_B8 = OFF_A + SA * A_STAGE;
constexpr int OFF_BP = OFF_B8 + S8 * B8_STAGE;
constexpr int OFF_SW = OFF_BP + SB * BP_STAGE;
constexpr int OFF_BAR = OFF_SW + SS * SW_STAGE;
constexpr int BNG = 64;          // GROUPED: accumulator columns per group = most rows of an item (MMA N); 8 buffers of 64 columns,
                                 // i.e. two K-tiles of accumulators in tensor memory: K-tile j+1's MMAs run while j is fetched
constexpr int KD = 12;           // K-tile-done ring (GROUPED): a multiple of SA and S8, deeper than any role can lag
constexpr int NUM_BARS = 2 * (SA + SB + S8 + SS + TB) + KD;
constexpr int OFF_TMEM = OFF_BAR + NUM_BARS * 8;
constexpr int SMEM_BYTES = OFF_TMEM + 16 + 1024;  // + slack to align the base to 1024 B

// Device error codes (w4a8_device_status detail): 0x100 | role << 4 | which wait.
enum : unsigned { ERR_PRODUCER = 0x110, ERR_MMA = 0x120, ERR_DEQUANT = 0x130, ERR_EPILOGUE = 0x140 };

struct Ring {
    int stage = 0;
    uint32_t phase = 0;
    const int depth;
    __device__ explicit Ring(int d) : depth(d) {}
    __device__ __forceinline__ void advance() {
        if (++stage == depth) { stage = 0; phase ^= 1u; }
    }
};

// ---- epilogue arithmetic on one chunk of NC accumulator columns ------------------------------------
// d[j] = 16 * D[m, n_j, b] (int32 from tensor memory), x = xs[m,b], sw16[j] = sw[n_j,b] / 16.
// Evaluates t = (float)d * x (rounded), acc = fma(t, sw16, acc): bit-identical to the reference's
// (float)c * xs * sw accumulation (kernels/gemm_mmq.cuh:104-105) because the two factors of 16 are exact.
//   EPI bit 0: int -> float by adding the integer to the bit pattern of 1.5 * 2^23 and subtracting that
//              constant as a float (exact for |d| < 2^22; here |d| <= 520,192) instead of cvt.rn.f32.s32
//   EPI bit 1: packed two-wide fp32 multiply / fma (mul.rn.f32x2, fma.rn.f32x2): same IEEE results per lane
__device__ __forceinline__ float cvt_exact(uint32_t d, bool magic) {
    if (magic) return __int_as_float((int)d + 0x4B400000) - 12582912.0f;
    return __int2float_rn((int)d);
}
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
template <int EPI, int NC>
__device__ __forceinline__ void epi_chunk(const uint32_t (&d)[NC], float x, const float *__restrict__ sw16, float *__restrict__ acc) {
    constexpr bool PACKED = (EPI & 2) != 0, MIXED = (EPI & 4) != 0;
    if (PACKED) {
        const uint64_t xx = pack_f32x2(x, x);
#pragma unroll
        for (int j4 = 0; j4 < NC / 4; j4++) {
            const float4 s4 = *reinterpret_cast<const float4 *>(sw16 + j4 * 4);
            // EPI bit 2: alternate between the two conversions so that neither the conversion pipe nor the
            // fp32 pipe carries all of them
            const bool MAGIC = MIXED ? ((j4 & 1) != 0) : ((EPI & 1) != 0);
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int j = j4 * 4 + 2 * h;
                uint64_t f2;
                if (MAGIC) {
                    const uint64_t i2 = pack_f32x2(__int_as_float((int)d[j] + 0x4B400000), __int_as_float((int)d[j + 1] + 0x4B400000));
                    const uint64_t c2 = pack_f32x2(-12582912.0f, -12582912.0f);
                    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(f2) : "l"(i2), "l"(c2));
                } else {
                    f2 = pack_f32x2(__int2float_rn((int)d[j]), __int2float_rn((int)d[j + 1]));
                }
                const uint64_t s2 = h == 0 ? pack_f32x2(s4.x, s4.y) : pack_f32x2(s4.z, s4.w);
                uint64_t a2 = pack_f32x2(acc[j], acc[j + 1]);
                uint64_t t2;
                asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(t2) : "l"(f2), "l"(xx));
                asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a2) : "l"(t2), "l"(s2));
                unpack_f32x2(a2, acc[j], acc[j + 1]);
            }
        }
    } else {
        constexpr bool MAGIC = (EPI & 1) != 0;
#pragma unroll
        for (int j4 = 0; j4 < NC / 4; j4++) {
            const float4 s4 = *reinterpret_cast<const float4 *>(sw16 + j4 * 4);
            const int j = j4 * 4;
            const float t0 = cvt_exact(d[j + 0], MAGIC) * x;
            const float t1 = cvt_exact(d[j + 1], MAGIC) * x;
            const float t2 = cvt_exact(d[j + 2], MAGIC) * x;
            const float t3 = cvt_exact(d[j + 3], MAGIC) * x;
            acc[j + 0] = fmaf(t0, s4.x, acc[j + 0]);
            acc[j + 1] = fmaf(t1, s4.y, acc[j + 1]);
            acc[j + 2] = fmaf(t2, s4.z, acc[j + 2]);
            acc[j + 3] = fmaf(t3, s4.w, acc[j + 3]);
        }
    }
}
// The same arithmetic with the roles of the two scales exchanged (grouped experts: lane = weight row, column = token):
// xs[j] belongs to column j, sw16 to the lane.  t = (float)d * xs (rounded), acc = fma(t, sw16, acc): the same operations
// on the same values as epi_chunk, so the same bits.
template <int NC>
__device__ __forceinline__ void epi_chunk_t(const uint32_t (&d)[NC], const float *__restrict__ xs, float sw16, uint64_t (&acc2)[NC / 2]) {
    // accumulators stay packed two to a 64-bit register across groups; the tokens' scales are read as packed pairs
    const uint64_t ss = pack_f32x2(sw16, sw16);
#pragma unroll
    for (int j4 = 0; j4 < NC / 4; j4++) {
        const ulonglong2 x = *reinterpret_cast<const ulonglong2 *>(xs + j4 * 4);   // {xs[4j4], xs[4j4+1]}, {xs[4j4+2], xs[4j4+3]}
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int j = j4 * 4 + 2 * h;
            const uint64_t f2 = pack_f32x2(__int2float_rn((int)d[j]), __int2float_rn((int)d[j + 1]));
            uint64_t t2;
            asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(t2) : "l"(f2), "l"(h == 0 ? x.x : x.y));
            asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[j / 2]) : "l"(t2), "l"(ss));
        }
    }
}
// Four consecutive scales of one row (one K-tile's worth) with one load; the address must be aligned to the
// size of the load.
__device__ __forceinline__ void load_scales4(const float *p, float (&v)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void load_scales4(const __half *p, float (&v)[4]) {
    const uint2 t = __ldg(reinterpret_cast<const uint2 *>(p));
    const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&t.x));
    const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&t.y));
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
// Debug path: the exact group dots of one chunk to Dout[m][n][b] (undoing the factor 16).
template <int NC>
__device__ __forceinline__ void epi_dump(const uint32_t (&d)[NC], int32_t *__restrict__ Dout, int m, int M, int ncol0, int N,
                                         int nb, int b) {
    if (m >= M) return;
#pragma unroll
    for (int j = 0; j < NC; j++) {
        const int n = ncol0 + j;
        if (n < N) Dout[((size_t)m * N + n) * nb + b] = ((int)d[j]) >> 4;
    }
}

// Grouped experts (GROUPED instantiation): the activation rows are sorted by expert, item i of the list says
// "expert x, sorted rows [y, y + z)" with z <= BNG (one item per 64-row tile of an expert, written on the device by
// moe_sort_kernel), the weights are the flat [experts * N][K/2] tensor of the reference (kernels/moe_fused.cuh:21-24:
// expert e starts e * N rows in), and one unit of work is (item, 128 of the expert's N outputs).
struct GroupList {
    const int4 *items = nullptr;
    const int *num_items = nullptr;
};

// One unit of work = (output tile, K split).  Tiles are numbered M-fastest so that CTAs running at the
// same time share weight tiles in L2; split s covers groups [s*gsplit, min(nb, (s+1)*gsplit)).
// Rows [m0, mend) of the tile are live; wrow0 is added to a column index to get its row in the weight tensor.
struct Work {
    int m0, mend, n0, wrow0, g0, g1, nkt, split;
};
template <bool GROUPED>
__device__ __forceinline__ Work decode_work(int w, int m_tiles, int num_tiles, int nb, int gsplit, int M, int N, int n_tiles,
                                            const GroupList &gl) {
    Work k;
    if (GROUPED) {
        const int4 it = __ldg(gl.items + w / n_tiles);
        k.split = 0;
        k.m0 = it.y;
        k.mend = it.y + it.z;
        k.n0 = (w % n_tiles) * BN;      // consecutive units share an item: its activation tile stays in L2
        k.wrow0 = it.x * N;
        k.g0 = 0;
        k.g1 = nb;
        k.nkt = (nb + GPK - 1) / GPK;
        return k;
    }
    const int tile = w % num_tiles;
    k.split = w / num_tiles;
    k.m0 = (tile % m_tiles) * BM;
    k.mend = M;
    k.n0 = (tile / m_tiles) * BN;
    k.wrow0 = 0;
    k.g0 = k.split * gsplit;
    k.g1 = min(nb, k.g0 + gsplit);
    const int ng = max(0, k.g1 - k.g0);
    k.nkt = (ng + GPK - 1) / GPK;
    return k;
}

// PEER (N-sharded weights, no split-K): every output tile is stored straight into EVERY rank's Y[M, ld] at its final
// columns (oa.col0 + n: plain 16-byte peer stores over NVLink) and the last CTA publishes the step's epoch, so the
// all-gather costs no extra pass over the outputs (peer_allgather.cuh).
template <typename ST, bool DUMP, int EPI, bool PEER = false, bool GROUPED = false>
__global__ void __launch_bounds__(THREADS, 1) gemm_w4a8_tc_kernel(
    const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
    const float *__restrict__ xs, const ST *__restrict__ sw, float *__restrict__ Y, int32_t *__restrict__ Dout,
    int M, int N, int K, int nsplit, int gsplit, const OutArgs oa, const GroupList gl) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw = ptx::smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char *base_ptr = smem_dyn + (base - raw);

    const uint32_t bar0 = base + OFF_BAR;
    auto BAR = [&](int idx) { return bar0 + 8u * idx; };
    // barrier index map
    constexpr int A_FULL = 0, A_EMPTY = A_FULL + SA, BP_FULL = A_EMPTY + SA, BP_EMPTY = BP_FULL + SB,
                  B8_FULL = BP_EMPTY + SB, B8_EMPTY = B8_FULL + S8, SW_FULL = B8_EMPTY + S8, SW_EMPTY = SW_FULL + SS,
                  TM_FULL = SW_EMPTY + SS, TM_EMPTY = TM_FULL + TB, KT_DONE = TM_EMPTY + TB;
    // GROUPED: ONE tcgen05.commit per K-tile instead of six (accumulator ready x 4, activation stage free, operand stage
    // free).  K-tile j of the CTA (counted across work units, the same in every role) commits to KT_DONE[j % KD]; whoever
    // needs "the MMAs of K-tile j have completed" waits for parity (j / KD) & 1 — the epilogue for its accumulators, the
    // producer and the expansion warps for the stages K-tile j read.  The epilogue then fetches all of a K-tile's live
    // columns in one go and hands the four accumulator buffers back together (MoE block at M = 512: 555 -> 530 us).
    constexpr bool KT_COMMIT = GROUPED;
    auto kt_done_wait = [&](int j) { return ptx::mbar_wait(BAR(KT_DONE + j % KD), (uint32_t)(j / KD) & 1u); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + OFF_TMEM);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = K / QBLK;
    const bool scales_aligned = ((reinterpret_cast<uintptr_t>(xs) & 15) == 0) && ((reinterpret_cast<uintptr_t>(sw) & (4 * sizeof(ST) - 1)) == 0);
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const int num_tiles = m_tiles * n_tiles;
    const int num_work = GROUPED ? *gl.num_items * n_tiles : num_tiles * nsplit;

    if (tid == 0) {
        for (int i = 0; i < SA; i++) { ptx::mbar_init(BAR(A_FULL + i), 1); ptx::mbar_init(BAR(A_EMPTY + i), 1); }
        for (int i = 0; i < SB; i++) { ptx::mbar_init(BAR(BP_FULL + i), 1); ptx::mbar_init(BAR(BP_EMPTY + i), DEQ_WARPS); }
        for (int i = 0; i < S8; i++) { ptx::mbar_init(BAR(B8_FULL + i), DEQ_WARPS); ptx::mbar_init(BAR(B8_EMPTY + i), 1); }
        for (int i = 0; i < SS; i++) { ptx::mbar_init(BAR(SW_FULL + i), DEQ_WARPS); ptx::mbar_init(BAR(SW_EMPTY + i), EPI_WARPS); }
        for (int i = 0; i < TB; i++) { ptx::mbar_init(BAR(TM_FULL + i), 1); ptx::mbar_init(BAR(TM_EMPTY + i), EPI_WARPS); }
        for (int i = 0; i < KD; i++) ptx::mbar_init(BAR(KT_DONE + i), 1);
        ptx::mbar_fence_init();
        ptx::tma_prefetch_desc(&tmA);
        ptx::tma_prefetch_desc(&tmB);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t *>(tmem_slot)), TB * BN);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            Ring ra(SA), rb(SB);
            bool ok = true;
            int kc = 0;
            for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
                const Work wk = decode_work<GROUPED>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gl);
                const int m0 = wk.m0, n0 = wk.n0;
                for (int kt = 0; kt < wk.nkt && ok; kt++, kc++) {
                    const int kbyte = (wk.g0 + kt * GPK) * QBLK;   // first K element of this K-tile (multiple of 32)
                    if (KT_COMMIT ? (kc >= SA && !kt_done_wait(kc - SA)) : !ptx::mbar_wait(BAR(A_EMPTY + ra.stage), ra.phase ^ 1u)) { dev_set_error(ERR_PRODUCER | 1); ok = false; break; }
                    ptx::mbar_arrive_expect_tx(BAR(A_FULL + ra.stage), A_STAGE);
                    ptx::tma_load_2d(base + OFF_A + ra.stage * A_STAGE, &tmA, kbyte, m0, BAR(A_FULL + ra.stage));
                    ra.advance();
                    if (!ptx::mbar_wait(BAR(BP_EMPTY + rb.stage), rb.phase ^ 1u)) { dev_set_error(ERR_PRODUCER | 2); ok = false; break; }
                    ptx::mbar_arrive_expect_tx(BAR(BP_FULL + rb.stage), BP_STAGE);
                    ptx::tma_load_2d(base + OFF_BP + rb.stage * BP_STAGE, &tmB, kbyte / 2, wk.wrow0 + n0, BAR(BP_FULL + rb.stage));
                    rb.advance();
                }
            }
            if (!ok) {  // give copies already in flight time to land before the CTA's shared memory goes away
                const long long t0 = clock64();
                while (clock64() - t0 < (1ll << 21)) { }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            Ring ra(SA), r8(S8), rt(TB);
            const uint32_t idesc = ptx::umma_idesc_s8(BM, BN), idesc_g = ptx::umma_idesc_s8(BN, BNG);
            bool ok = true;
            int kc = 0;
            for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
                const Work wk = decode_work<GROUPED>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gl);
                for (int kt = 0; kt < wk.nkt && ok; kt++, kc++) {
                    if (!ptx::mbar_wait(BAR(A_FULL + ra.stage), ra.phase)) { dev_set_error(ERR_MMA | 1); ok = false; break; }
                    if (!ptx::mbar_wait(BAR(B8_FULL + r8.stage), r8.phase)) { dev_set_error(ERR_MMA | 2); ok = false; break; }
                    ptx::tc_fence_after_sync();
                    const uint64_t adesc = ptx::umma_desc_k_sw128(base + OFF_A + ra.stage * A_STAGE);
                    const uint64_t bdesc = ptx::umma_desc_k_sw128(base + OFF_B8 + r8.stage * B8_STAGE);
                    const int ng = min(GPK, wk.g1 - (wk.g0 + kt * GPK));
                    if (KT_COMMIT) {
                        // K-tile kc uses the accumulator half kc & 1 (GPK buffers of BNG columns); wait until the epilogue has
                        // fetched the K-tile that used it before (kc - 2), then the K-tile's MMAs back to back and ONE commit
                        const int half = kc & 1;
                        if (!ptx::mbar_wait(BAR(TM_EMPTY + half), ((uint32_t)(kc >> 1) & 1u) ^ 1u)) { dev_set_error(ERR_MMA | 3); ok = false; break; }
                        ptx::tc_fence_after_sync();
                        for (int g = 0; g < ng; g++) {
                            // the expanded weights are the MMA's A operand (accumulator lanes = weight rows), the activations
                            // its B operand (columns = tokens, BNG of them): an expert's tile has few live tokens, and the
                            // epilogue's work follows the live COLUMNS while all 128 lanes stay busy
                            ptx::umma_i8(tmem_base + (half * GPK + g) * BNG, bdesc + (uint64_t)(g * 2), adesc + (uint64_t)(g * 2), idesc_g, 0u);
                        }
                        ptx::umma_commit(BAR(KT_DONE + kc % KD));
                        ra.advance();
                        r8.advance();
                        continue;
                    }
                    for (int g = 0; g < ng; g++) {
                        if (!ptx::mbar_wait(BAR(TM_EMPTY + rt.stage), rt.phase ^ 1u)) { dev_set_error(ERR_MMA | 3); ok = false; break; }
                        ptx::tc_fence_after_sync();
                        // group g = bytes [32g, 32g+32) of every 128-byte operand row: advance the start address
                        ptx::umma_i8(tmem_base + rt.stage * BN, adesc + (uint64_t)(g * 2), bdesc + (uint64_t)(g * 2), idesc, 0u);
                        ptx::umma_commit(BAR(TM_FULL + rt.stage));
                        rt.advance();
                    }
                    ptx::umma_commit(BAR(A_EMPTY + ra.stage));
                    ptx::umma_commit(BAR(B8_EMPTY + r8.stage));
                    ra.advance();
                    r8.advance();
                }
            }
        }
    } else if (warp < 2 + DEQ_WARPS) {
        // ---------------- int4 -> int8 expansion + weight-scale staging ----------------
        const int dt = tid - 64;  // 0..DEQ_WARPS*32-1
        Ring rb(SB), r8(S8), rs(SS);
        bool ok = true;
        int kc = 0;
        for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
            const Work wk = decode_work<GROUPED>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gl);
            const int n0 = wk.n0;
            if (GROUPED && dt == 0 && scales_aligned) {
                // An expert's scales are touched by this CTA only, so every K-tile's scale loads would wait for HBM (with
                // dense weights another CTA has usually brought them into L2).  The scale rows of a unit are one contiguous
                // block each: ask for the NEXT unit's blocks now (and for this CTA's first unit at its start).
                auto prefetch_unit = [&](const Work &u) {
                    const int nrows = min(BN, N - u.n0), mrows = u.mend - u.m0;
                    const uint32_t wbytes = (uint32_t)((size_t)nrows * nb * sizeof(ST)) & ~15u, xbytes = (uint32_t)((size_t)mrows * nb * 4) & ~15u;
                    const ST *wp = sw + (size_t)(u.wrow0 + u.n0) * nb;
                    const float *xp = xs + (size_t)u.m0 * nb;
                    if (wbytes && (reinterpret_cast<uintptr_t>(wp) & 15) == 0) ptx::prefetch_l2_bulk(wp, wbytes);
                    if (xbytes && (reinterpret_cast<uintptr_t>(xp) & 15) == 0) ptx::prefetch_l2_bulk(xp, xbytes);
                };
                if (wi == (int)blockIdx.x) prefetch_unit(wk);
                if (wi + (int)gridDim.x < num_work) prefetch_unit(decode_work<GROUPED>(wi + gridDim.x, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gl));
            }
            for (int kt = 0; kt < wk.nkt && ok; kt++, kc++) {
                // ---- this K-tile's scales: issue the loads first, they complete behind the expansion below.
                // A row's GPK scales are contiguous in memory: one 16-byte (fp32) or 8-byte (fp16) load per row
                // when the K-tile is complete and the addresses line up, else element by element.
                constexpr int RW = BN / (DEQ_WARPS * 32), RX = BM / (DEQ_WARPS * 32);
                const int b0 = wk.g0 + kt * GPK;   // first group of this K-tile
                const bool vec = !DUMP && (b0 + GPK <= wk.g1) && (nb % GPK == 0) && (b0 % GPK == 0) && scales_aligned;
                float vw[RW][GPK], vx[RX][GPK];
#pragma unroll
                for (int r = 0; r < RW; r++) {
                    const int n = n0 + dt + r * DEQ_WARPS * 32;
#pragma unroll
                    for (int g = 0; g < GPK; g++) vw[r][g] = 0.f;
                    if (!DUMP && n < N) {
                        const ST *swrow = sw + (size_t)(wk.wrow0 + n) * nb;
                        if (vec) load_scales4(swrow + b0, vw[r]);
                        else {
#pragma unroll
                            for (int g = 0; g < GPK; g++)
                                if (b0 + g < wk.g1) vw[r][g] = sval(swrow[b0 + g]);
                        }
                    }
                }
#pragma unroll
                for (int r = 0; r < RX; r++) {
                    const int m = wk.m0 + dt + r * DEQ_WARPS * 32;
#pragma unroll
                    for (int g = 0; g < GPK; g++) vx[r][g] = 0.f;
                    if (!DUMP && m < wk.mend) {
                        if (vec) load_scales4(xs + (size_t)m * nb + b0, vx[r]);
                        else {
#pragma unroll
                            for (int g = 0; g < GPK; g++)
                                if (b0 + g < wk.g1) vx[r][g] = xs[(size_t)m * nb + b0 + g];
                        }
                    }
                }

                // ---- expansion of the packed stage into the operand stage
                bool w = ptx::mbar_wait_warp(BAR(BP_FULL + rb.stage), rb.phase) && (KT_COMMIT ? (kc < S8 || ptx::mbar_wait_warp(BAR(KT_DONE + (kc - S8) % KD), (uint32_t)((kc - S8) / KD) & 1u))
                                                                                                   : ptx::mbar_wait_warp(BAR(B8_EMPTY + r8.stage), r8.phase ^ 1u));
                if (!w) { dev_set_error(ERR_DEQUANT | 1); ok = false; break; }
                const unsigned char *src = base_ptr + OFF_BP + rb.stage * BP_STAGE;
                unsigned char *dst = base_ptr + OFF_B8 + r8.stage * B8_STAGE;
                // All loads first, then expansion and stores: the compiler cannot tell that the two stages do not
                // overlap, so in one loop every load would wait for the previous store.
                constexpr int NT = (BN * 8) / (DEQ_WARPS * 32);
                uint2 pk[NT];
#pragma unroll
                for (int i = 0; i < NT; i++) {
                    const int j = dt + i * DEQ_WARPS * 32;
                    const int n = j >> 3, c = j & 7;  // row n, 8 packed bytes = 16 weights = one 16-byte chunk
                    pk[i] = *reinterpret_cast<const uint2 *>(src + n * (KT / 2) + c * 8);
                }
#pragma unroll
                for (int i = 0; i < NT; i++) {
                    const int j = dt + i * DEQ_WARPS * 32;
                    const int n = j >> 3, c = j & 7;
                    uint4 o;
                    unpack8_x16_seq(pk[i].x, o.x, o.y);
                    unpack8_x16_seq(pk[i].y, o.z, o.w);
                    *reinterpret_cast<uint4 *>(dst + n * KT + ((c ^ (n & 7)) << 4)) = o;
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) { ptx::mbar_arrive(BAR(B8_FULL + r8.stage)); ptx::mbar_arrive(BAR(BP_EMPTY + rb.stage)); }
                rb.advance();
                r8.advance();

                // ---- store the scales: weight scales transposed to [group][n] and pre-multiplied by the exact
                // 1/16 that undoes the 16x of the expansion, activation scales transposed to [group][m]
                w = ptx::mbar_wait_warp(BAR(SW_EMPTY + rs.stage), rs.phase ^ 1u);
                if (!w) { dev_set_error(ERR_DEQUANT | 2); ok = false; break; }
                float *ssw = reinterpret_cast<float *>(base_ptr + OFF_SW + rs.stage * SW_STAGE);
                float *ssx = ssw + GPK * BN;
#pragma unroll
                for (int r = 0; r < RW; r++)
#pragma unroll
                    for (int g = 0; g < GPK; g++) ssw[g * BN + dt + r * DEQ_WARPS * 32] = vw[r][g] * 0.0625f;
#pragma unroll
                for (int r = 0; r < RX; r++)
#pragma unroll
                    for (int g = 0; g < GPK; g++) ssx[g * BM + dt + r * DEQ_WARPS * 32] = vx[r][g];
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(BAR(SW_FULL + rs.stage));
                rs.advance();
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int ew = warp - (2 + DEQ_WARPS);  // 0..EPI_WARPS-1
        const int quad = warp & 3;              // TMEM lanes [32*quad, 32*quad+32) are the ones this warp may read
        const int col0 = (ew >> 2) * EPI_COLS;  // this warp's accumulator columns [col0, col0 + EPI_COLS)
        Ring rs(SS), rt(TB);
        bool ok = true;
        if (GROUPED) {
            // Transposed accumulator: lanes are weight rows (all 128 live), columns are the item's tokens (z <= BNG live, 32
            // on average).  The 4 warps that share a quad of lanes deal the live columns out in chunks of CW: warp group cg
            // takes chunks cg and cg + 4, so that at z = 32 every one of the 16 warps converts and scales 8 columns per
            // group.  A K-tile's accumulators (one half of tensor memory) are handed back once all of its groups have been
            // fetched; the other half is being written by the next K-tile's MMAs meanwhile.
            constexpr int CW = 8, CK = BNG / (4 * CW);     // 2 chunks of 8 columns per warp at most
            const int cg = ew >> 2;
            int kce = 0;                                   // K-tiles of this CTA so far (the index every role counts)
            for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
                const Work wk = decode_work<GROUPED>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gl);
                const int z = wk.mend - wk.m0;
                const int nlive = z > CW * cg ? (z - CW * cg - 1) / (4 * CW) + 1 : 0;   // chunk k covers columns CW*(cg + 4k) ...
                const int n = wk.n0 + quad * 32 + lane;
                uint64_t acc[CK][CW / 2];                              // packed pairs of fp32 accumulators
#pragma unroll
                for (int k = 0; k < CK; k++)
#pragma unroll
                    for (int j = 0; j < CW / 2; j++) acc[k][j] = 0ull;
                const int ngroups = wk.g1 - wk.g0;
                for (int gi = 0; gi < ngroups; gi += GPK) {             // one K-tile = up to GPK groups = one commit
                    const int ngk = min(GPK, ngroups - gi);
                    if (!ptx::mbar_wait_warp(BAR(SW_FULL + rs.stage), rs.phase)) { dev_set_error(ERR_EPILOGUE | 1); ok = false; break; }
                    const float *stage = reinterpret_cast<const float *>(base_ptr + OFF_SW + rs.stage * SW_STAGE);
                    if (!ptx::mbar_wait_warp(BAR(KT_DONE + kce % KD), (uint32_t)(kce / KD) & 1u)) { dev_set_error(ERR_EPILOGUE | 2); ok = false; break; }
                    ptx::tc_fence_after_sync();
                    const int half = kce & 1;
                    kce++;
                    const uint32_t tl = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(half * GPK * BNG + CW * cg);
                    // Fetches are issued in batches of four chunks (32 registers) with one wait per batch, the K-tile's half of
                    // tensor memory is handed back after the last fetch, and the loops are fully unrolled per case (one or two
                    // chunks per group): the epilogue is bound by its instruction count, not by the arithmetic in it.
                    auto release = [&]() {
                        ptx::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(BAR(TM_EMPTY + half));
                    };
                    const float *xs0 = stage + GPK * BN + CW * cg;          // + g * BM (+ 4 * CW for the second chunk)
                    const float *sw0 = stage + quad * 32 + lane;            // + g * BN
                    uint32_t d[4][CW];
                    if (nlive == 0) {
                        release();
                    } else if (nlive == 1) {
#pragma unroll
                        for (int g = 0; g < GPK; g++)
                            if (g < ngk) ptx::tmem_ld(tl + g * BNG, d[g]);
                        ptx::tmem_ld_wait();
                        release();
#pragma unroll
                        for (int g = 0; g < GPK; g++)
                            if (g < ngk) epi_chunk_t<CW>(d[g], xs0 + g * BM, sw0[g * BN], acc[0]);
                    } else {
#pragma unroll
                        for (int h = 0; h < GPK / 2; h++) {                 // groups 2h and 2h + 1, both chunks of each
                            const int g0 = 2 * h, g1 = 2 * h + 1;
                            if (g0 < ngk) { ptx::tmem_ld(tl + g0 * BNG, d[0]); ptx::tmem_ld(tl + g0 * BNG + 4 * CW, d[1]); }
                            if (g1 < ngk) { ptx::tmem_ld(tl + g1 * BNG, d[2]); ptx::tmem_ld(tl + g1 * BNG + 4 * CW, d[3]); }
                            ptx::tmem_ld_wait();
                            if (h == GPK / 2 - 1) release();
                            if (g0 < ngk) {
                                const float swl = sw0[g0 * BN];
                                epi_chunk_t<CW>(d[0], xs0 + g0 * BM, swl, acc[0]);
                                epi_chunk_t<CW>(d[1], xs0 + g0 * BM + 4 * CW, swl, acc[1]);
                            }
                            if (g1 < ngk) {
                                const float swl = sw0[g1 * BN];
                                epi_chunk_t<CW>(d[2], xs0 + g1 * BM, swl, acc[0]);
                                epi_chunk_t<CW>(d[3], xs0 + g1 * BM + 4 * CW, swl, acc[1]);
                            }
                            if (h == 0) ptx::tc_fence_after_sync();
                        }
                    }
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(BAR(SW_EMPTY + rs.stage));
                    rs.advance();
                }
                if (!ok) break;
                if (n < N) {   // consecutive lanes write consecutive floats of a row of Y
#pragma unroll
                    for (int k = 0; k < CK; k++)
#pragma unroll
                        for (int j = 0; j < CW; j += 2) {
                            const int col = CW * (cg + 4 * k) + j;
                            float lo, hi;
                            unpack_f32x2(acc[k][j / 2], lo, hi);
                            if (k < nlive && col < z) Y[(size_t)(wk.m0 + col) * N + n] = lo;
                            if (k < nlive && col + 1 < z) Y[(size_t)(wk.m0 + col + 1) * N + n] = hi;
                        }
                }
            }
        }
        for (int wi = blockIdx.x; !GROUPED && wi < num_work && ok; wi += gridDim.x) {
            const Work wk = decode_work<GROUPED>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gl);
            const int m0 = wk.m0, n0 = wk.n0;
            const int m = m0 + quad * 32 + lane;
            // a warp whose 32 rows all lie beyond M only keeps the barriers moving
            const bool rows_live = (m0 + quad * 32) < wk.mend;
            float acc[EPI_COLS];
#pragma unroll
            for (int j = 0; j < EPI_COLS; j++) acc[j] = 0.f;
            const int ngroups = wk.g1 - wk.g0;
            const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16) + col0;
            // One flat loop over the groups of this unit of work.  The 2 chunks (EPI_CH columns each) of a group
            // are software-pipelined with the next group's: the tcgen05.ld of the next chunk is in flight while
            // the current one is converted and accumulated.  d0 holds the first half of this warp's columns of
            // a group, d1 the second.  Both scales come from the staged K-tile slice in shared memory, so the
            // loop issues no global loads.
            uint32_t d0[EPI_CH], d1[EPI_CH];
            const float *ssw = nullptr, *ssx = nullptr;
            bool w = true;
            if (ngroups > 0) {   // a split beyond the last group has no work: its partial sums are zeros
                w = ptx::mbar_wait_warp(BAR(TM_FULL + rt.stage), rt.phase);
                if (!w) { dev_set_error(ERR_EPILOGUE | 2); ok = false; break; }
                ptx::tc_fence_after_sync();
                if (rows_live) ptx::tmem_ld(tlane + rt.stage * BN, d0);
            }
#pragma unroll EPI_UNROLL
            for (int gi = 0; gi < ngroups; gi++) {
                const int g = gi & (GPK - 1);
                if (g == 0) {
                    w = ptx::mbar_wait_warp(BAR(SW_FULL + rs.stage), rs.phase);
                    if (!w) { dev_set_error(ERR_EPILOGUE | 1); ok = false; break; }
                    ssw = reinterpret_cast<const float *>(base_ptr + OFF_SW + rs.stage * SW_STAGE) + col0;
                    ssx = reinterpret_cast<const float *>(base_ptr + OFF_SW + rs.stage * SW_STAGE) + GPK * BN + quad * 32 + lane;
                }
                const float x = ssx[g * BM];
                const uint32_t tcur = tlane + rt.stage * BN;
                // ---- first half: wait for it, start the second half's load, then compute
                ptx::tmem_ld_wait();
                if (rows_live) ptx::tmem_ld(tcur + EPI_CH, d1);
                if (rows_live) {
                    if (DUMP) epi_dump<EPI_CH>(d0, Dout, m, wk.mend, n0 + col0, N, nb, wk.g0 + gi);
                    else epi_chunk<EPI, EPI_CH>(d0, x, ssw + g * BN, acc);
                }
                // ---- second half: wait, release the accumulator buffer, start the next group's load
                ptx::tmem_ld_wait();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(BAR(TM_EMPTY + rt.stage));
                rt.advance();
                if (gi + 1 < ngroups) {
                    w = ptx::mbar_wait_warp(BAR(TM_FULL + rt.stage), rt.phase);
                    if (!w) { dev_set_error(ERR_EPILOGUE | 3); ok = false; break; }
                    ptx::tc_fence_after_sync();
                    if (rows_live) ptx::tmem_ld(tlane + rt.stage * BN, d0);
                }
                if (rows_live) {
                    if (DUMP) epi_dump<EPI_CH>(d1, Dout, m, wk.mend, n0 + col0 + EPI_CH, N, nb, wk.g0 + gi);
                    else epi_chunk<EPI, EPI_CH>(d1, x, ssw + g * BN + EPI_CH, acc + EPI_CH);
                }
                if (g == GPK - 1 || gi + 1 == ngroups) {   // done with this K-tile's scales
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(BAR(SW_EMPTY + rs.stage));
                    rs.advance();
                }
            }
            if (!ok) break;
            if (!DUMP && ok && m < wk.mend) {
                const int nleft = N - (n0 + col0);
                const int targets = PEER ? oa.peers->world : 1;
                for (int k = 0; k < targets; k++) {
                    if (PEER && oa.local_only && k != oa.peers->rank) continue;
                    float *yrow = PEER ? reinterpret_cast<float *>(oa.peers->base[k] + oa.y_off) + (size_t)m * oa.ld + oa.col0 + n0 + col0
                                       : Y + (size_t)wk.split * ((size_t)M * N) + (size_t)m * N + n0 + col0;
                    if (nleft >= EPI_COLS && ((reinterpret_cast<uintptr_t>(yrow) & 15) == 0)) {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; j += 4)
                            *reinterpret_cast<float4 *>(yrow + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; j++)
                            if (j < nleft) yrow[j] = acc[j];
                    }
                }
            }
        }
    }

    publish_out<PEER>(oa, warp >= 2 + DEQ_WARPS);
    // ---------------- teardown ----------------
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TB * BN);
    }
}

// Adds the split-K partial sums in ascending split order (the order of the reference's
// reduce_splitk_kernel, kernels/gemm_mmq.cuh:201-204): Y[i] = ((0 + P0[i]) + P1[i]) + ...
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float *__restrict__ P, float *__restrict__ Y, long MN, int nsplit) {
    const long stride = (long)gridDim.x * blockDim.x;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < MN; i += stride) {
        float s = 0.f;
        for (int sp = 0; sp < nsplit; sp++) s += P[(size_t)sp * MN + i];
        Y[i] = s;
    }
}

// ---- host side ------------------------------------------------------------------------------------
// experts > 0: grouped launch (GROUPED instantiation): M = sorted activation rows, N = outputs per expert, Wq / sw the
// flat tensors of `experts` experts, gl the item list; max_items bounds the list's length (grid size only).
template <typename ST, bool DUMP, int EPI, bool PEER = false, bool GROUPED = false>
inline int launch_tc_e(const int8_t *X, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int32_t *D,
                       int M, int N, int K, int nsplit, int gsplit, cudaStream_t st, const OutArgs &oa,
                       const GroupList &gl = GroupList(), int experts = 0, int max_items = 0) {
    CUtensorMap tmA, tmB;
    int rc = make_tmap_u8(&tmA, X, (uint64_t)K, (uint64_t)M, KT, BM, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != W4A8_OK) return rc;
    rc = make_tmap_u8(&tmB, Wq, (uint64_t)K / 2, (uint64_t)N * (GROUPED ? experts : 1), KT / 2, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != W4A8_OK) return rc;
    auto kern = gemm_w4a8_tc_kernel<ST, DUMP, EPI, PEER, GROUPED>;
    static PerDevice<bool> configured_dev;              // the opt-in is a per-device function attribute
    bool &configured = configured_dev.get();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return cuda_fail(e, "gemm smem opt-in");
        configured = true;
    }
    const long tiles = GROUPED ? (long)max_items * ((N + BN - 1) / BN) : (long)((M + BM - 1) / BM) * ((N + BN - 1) / BN) * nsplit;
    const int sms = sm_count();
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(tmA, tmB, xs, sw, Y, D, M, N, K, nsplit, gsplit, PEER ? oa : OutArgs(), gl);
    return launch_status("gemm_w4a8_tc");
}

// Grouped experts: Y[sorted row, n] for the rows and experts the item list names (rows of experts without an item,
// and rows no item covers, are not written).  Same arithmetic per (row, expert) as launch_tc.
inline int launch_tc_grouped(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int rows, int N, int K,
                             int scale_dtype, int experts, const GroupList &gl, int max_items, cudaStream_t st) {
    if (scale_dtype == 1)
        return launch_tc_e<__half, false, 2, false, true>(X, xs, Wq, (const __half *)sw, Y, nullptr, rows, N, K, 1, K / QBLK, st, OutArgs(), gl, experts, max_items);
    return launch_tc_e<float, false, 2, false, true>(X, xs, Wq, (const float *)sw, Y, nullptr, rows, N, K, 1, K / QBLK, st, OutArgs(), gl, experts, max_items);
}

// Needs X and Wq 16-byte aligned (TMA global address rule); the caller checks.
// Epilogue arithmetic variant (see epi_chunk): all variants give identical bits.  W4A8_GEMM_EPI overrides the
// default for measurements (0 cvt, 1 magic-number conversion, 2 cvt + f32x2, 3 magic + f32x2).
inline int epi_variant() {
    static int v = -1;
    if (v < 0) {
        const char *e = getenv("W4A8_GEMM_EPI");
        v = e ? atoi(e) & 7 : 2;
    }
    return v;
}
template <typename ST, bool DUMP>
inline int launch_tc_t(const int8_t *X, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int32_t *D,
                       int M, int N, int K, int nsplit, int gsplit, cudaStream_t st, const OutArgs &oa) {
    if (!DUMP && oa.peers) return launch_tc_e<ST, false, 2, true>(X, xs, Wq, sw, Y, D, M, N, K, nsplit, gsplit, st, oa);
    switch (DUMP ? 0 : epi_variant()) {
        case 1: return launch_tc_e<ST, DUMP, 1>(X, xs, Wq, sw, Y, D, M, N, K, nsplit, gsplit, st, oa);
        case 2: return launch_tc_e<ST, DUMP, 2>(X, xs, Wq, sw, Y, D, M, N, K, nsplit, gsplit, st, oa);
        case 3: return launch_tc_e<ST, DUMP, 3>(X, xs, Wq, sw, Y, D, M, N, K, nsplit, gsplit, st, oa);
        case 6: return launch_tc_e<ST, DUMP, 6>(X, xs, Wq, sw, Y, D, M, N, K, nsplit, gsplit, st, oa);
        default: return launch_tc_e<ST, DUMP, 0>(X, xs, Wq, sw, Y, D, M, N, K, nsplit, gsplit, st, oa);
    }
}

// nsplit = 1: Y is the output.  nsplit > 1: Y is the [nsplit][M][N] partial-sum workspace and gsplit the
// number of groups per split.
inline int launch_tc(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int M, int N, int K,
                     int scale_dtype, int nsplit, int gsplit, cudaStream_t st, const OutArgs &oa = OutArgs()) {
    if (scale_dtype == 1)
        return launch_tc_t<__half, false>(X, xs, Wq, (const __half *)sw, Y, nullptr, M, N, K, nsplit, gsplit, st, oa);
    return launch_tc_t<float, false>(X, xs, Wq, (const float *)sw, Y, nullptr, M, N, K, nsplit, gsplit, st, oa);
}
inline int launch_tc_dump(const int8_t *X, const uint8_t *Wq, int32_t *D, int M, int N, int K, cudaStream_t st) {
    return launch_tc_t<float, true>(X, nullptr, Wq, (const float *)nullptr, nullptr, D, M, N, K, 1, K / QBLK, st, OutArgs());
}

}  // namespace gemm
}  // namespace w4a8
