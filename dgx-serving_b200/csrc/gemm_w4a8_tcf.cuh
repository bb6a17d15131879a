// W4A8 prefill / verify GEMM, second formulation: the group dots come out of the tensor core as FLOATS.
//
// Why.  With int8 operands (gemm_w4a8_tc.cuh, tcgen05 kind::i8) every (m, n, group) needs an int32 -> fp32
// conversion on the CUDA cores before the two scale multiplications, and that conversion runs at a quarter of the
// fp32 rate on this part: it, not the tensor core, sets the pace.  The integer operands are small — activations in
// [-127, 127], weights in [-8, 7] — so both are EXACT in fp16, every product is exact in fp32, and the sum of the 32
// products of a group (|sum| <= 32,512) is exact in fp32 in any order.  tcgen05.mma kind::f16 with fp32 accumulation
// therefore returns exactly (float)D[m,n,b], bit for bit the value the reference computes with
// mma.sync ... s32 followed by a conversion (kernels/gemm_mmq.cuh:98-105).  What remains per (m, n, group) is
// t = D * xs[m,b]; acc = fma(t, sw[n,b], acc), done two-wide (mul.f32x2 / fma.f32x2): same order, same bits.
//
// Same structure as the int8 kernel: persistent, 1 CTA/SM, 128x128 tile, K-tile of 128 elements = 4 groups:
//   warp 0      TMA producer: raw int8 activations [128 x 128 B] and packed int4 weights [128 x 64 B]
//   warp 1      MMA issuer: per group two tcgen05.mma kind::f16 (128x128x16 each; the second accumulates) into one of
//               four 128-column fp32 accumulator buffers in tensor memory
//   warps 2-5   conversion: int8 -> fp16 and int4 -> fp16 into the two K-major, 128-byte-swizzled operand stages
//               (each 2 swizzle atoms of 64 elements), plus the weight scales of the K-tile transposed to [group][n]
//   warps 6-13  epilogue: tcgen05.ld (16-column chunks, software-pipelined), scale, accumulate, store
// Inside every 8-element chunk both operands are stored in the order 0,4,1,5,2,6,3,7 (what the cheapest nibble
// extraction produces); a dot product does not care as long as both sides agree.
#pragma once
#include <cuda.h>
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "gemm_w4a8_tc.cuh"   // Work / decode_work / Ring / pack_f32x2 / error codes

namespace w4a8 {
namespace gemmf {

using gemm::BM;
using gemm::BN;
using gemm::KT;
using gemm::GPK;
using gemm::Ring;
using gemm::Work;
using gemm::decode_work;

constexpr int SR = 3;                       // raw (TMA) stages
constexpr int SO = 2;                       // converted operand stages
constexpr int SS = 4;                       // weight-scale stages
constexpr int TB = 4;                       // TMEM accumulator buffers
constexpr int ARAW = BM * KT;               // 16 KB
constexpr int BRAW = BN * KT / 2;           // 8 KB
constexpr int ATOM = 128 * 128;             // one swizzle atom: 128 rows x 128 B (64 fp16)
constexpr int OPA = 2 * ATOM;               // 32 KB: activations of a K-tile in fp16
constexpr int OPB = 2 * ATOM;               // 32 KB: weights of a K-tile in fp16
constexpr int SW_STAGE = GPK * BN * 4;      // 2 KB
constexpr int CONV_WARPS = 4, EPI_WARPS = 8;
constexpr int THREADS = (2 + CONV_WARPS + EPI_WARPS) * 32;   // 448
constexpr int EPI_COLS = BN / (EPI_WARPS / 4);               // 64 accumulator columns per epilogue warp
constexpr int EPI_CH = 16;                                   // columns per tcgen05.ld
constexpr int OFF_OPA = 0;
constexpr int OFF_OPB = OFF_OPA + SO * OPA;
constexpr int OFF_ARAW = OFF_OPB + SO * OPB;
constexpr int OFF_BRAW = OFF_ARAW + SR * ARAW;
constexpr int OFF_SW = OFF_BRAW + SR * BRAW;
constexpr int OFF_BAR = OFF_SW + SS * SW_STAGE;
constexpr int NUM_BARS = 2 * (SR + SR + SO + SS + TB);
constexpr int OFF_TMEM = OFF_BAR + NUM_BARS * 8;
constexpr int SMEM_BYTES = OFF_TMEM + 16 + 1024;

// Instruction descriptor for kind::f16: D = fp32 (c_format 1, bits [4,6)); A, B = fp16 (format 0); K-major both;
// N >> 3 in [17,23); M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// ---- integer -> fp16 without a conversion instruction ----------------------------------------------------------
// An fp16 with exponent field 0x19 (bits 0x6400) has the value 1024 + mantissa: OR-ing an 8-bit unsigned integer u into
// the mantissa gives 1024 + u exactly, and one packed subtraction removes the offset.
// Eight packed int4 weights w (nibble i = element i) -> halves (e0,e4) (e1,e5) (e2,e6) (e3,e7), each = nibble - 8:
//   low-nibble pairs:  (w & 0x000F000F) | 0x64006400          = 1024 + n        -> minus 1032
//   high-nibble pairs: (w & 0x00F000F0) | 0x64006400          = 1024 + 16 n     -> times 1/16, minus 72   (one fma)
__device__ __forceinline__ uint4 w4_to_f16x8(uint32_t w) {
    const uint32_t MAGIC = 0x64006400u;
    const __half2 sub_lo = __halves2half2(__ushort_as_half(0x6408), __ushort_as_half(0x6408));   // 1032
    const __half2 mul_hi = __halves2half2(__ushort_as_half(0x2C00), __ushort_as_half(0x2C00));   // 1/16
    const __half2 add_hi = __halves2half2(__ushort_as_half(0xD480), __ushort_as_half(0xD480));   // -72
    const uint32_t w8 = w >> 8;
    uint32_t p0 = (w & 0x000F000Fu) | MAGIC, p1 = (w & 0x00F000F0u) | MAGIC;       // (e0,e4) (e1,e5)
    uint32_t p2 = (w8 & 0x000F000Fu) | MAGIC, p3 = (w8 & 0x00F000F0u) | MAGIC;     // (e2,e6) (e3,e7)
    __half2 h0 = __hsub2(*reinterpret_cast<__half2 *>(&p0), sub_lo);
    __half2 h1 = __hfma2(*reinterpret_cast<__half2 *>(&p1), mul_hi, add_hi);
    __half2 h2 = __hsub2(*reinterpret_cast<__half2 *>(&p2), sub_lo);
    __half2 h3 = __hfma2(*reinterpret_cast<__half2 *>(&p3), mul_hi, add_hi);
    return make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                      *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
}
// Eight int8 activations (x0..x3 in a, x4..x7 in b) -> halves (x0,x4) (x1,x5) (x2,x6) (x3,x7).  x ^ 0x80 = x + 128 as an
// unsigned byte; byte_perm puts byte i of a and of b into the low bytes of the two halves; 1024 + 128 is subtracted.
__device__ __forceinline__ uint4 i8_to_f16x8(uint32_t a, uint32_t b) {
    const __half2 sub = __halves2half2(__ushort_as_half(0x6480), __ushort_as_half(0x6480));      // 1152
    a ^= 0x80808080u;
    b ^= 0x80808080u;
    uint32_t p0 = (__byte_perm(a, b, 0x0400) & 0x00FF00FFu) | 0x64006400u;
    uint32_t p1 = (__byte_perm(a, b, 0x0501) & 0x00FF00FFu) | 0x64006400u;
    uint32_t p2 = (__byte_perm(a, b, 0x0602) & 0x00FF00FFu) | 0x64006400u;
    uint32_t p3 = (__byte_perm(a, b, 0x0703) & 0x00FF00FFu) | 0x64006400u;
    __half2 h0 = __hsub2(*reinterpret_cast<__half2 *>(&p0), sub), h1 = __hsub2(*reinterpret_cast<__half2 *>(&p1), sub);
    __half2 h2 = __hsub2(*reinterpret_cast<__half2 *>(&p2), sub), h3 = __hsub2(*reinterpret_cast<__half2 *>(&p3), sub);
    return make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                      *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
}
// Byte address, inside an operand stage, of the 16-byte chunk holding elements [8c, 8c+8) of row r (c = 0..15):
// swizzle atom c / 8, row pitch 128 B, chunk position (c % 8) ^ (r % 8).
__device__ __forceinline__ int op_chunk(int r, int c) { return (c >> 3) * ATOM + r * 128 + (((c & 7) ^ (r & 7)) << 4); }

// ---- epilogue arithmetic on NC accumulator columns (floats straight from tensor memory) ------------------------
template <int NC>
__device__ __forceinline__ void epi_chunk_f(const uint32_t (&d)[NC], float x, const float *__restrict__ swv, float *__restrict__ acc) {
    const uint64_t xx = gemm::pack_f32x2(x, x);
#pragma unroll
    for (int j4 = 0; j4 < NC / 4; j4++) {
        const float4 s4 = *reinterpret_cast<const float4 *>(swv + j4 * 4);
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int j = j4 * 4 + 2 * h;
            const uint64_t f2 = gemm::pack_f32x2(__uint_as_float(d[j]), __uint_as_float(d[j + 1]));
            const uint64_t s2 = h == 0 ? gemm::pack_f32x2(s4.x, s4.y) : gemm::pack_f32x2(s4.z, s4.w);
            uint64_t a2 = gemm::pack_f32x2(acc[j], acc[j + 1]);
            uint64_t t2;
            asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(t2) : "l"(f2), "l"(xx));
            asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a2) : "l"(t2), "l"(s2));
            gemm::unpack_f32x2(a2, acc[j], acc[j + 1]);
        }
    }
}
template <int NC>
__device__ __forceinline__ void epi_dump_f(const uint32_t (&d)[NC], int32_t *__restrict__ Dout, int m, int M, int ncol0, int N, int nb, int b) {
    if (m >= M) return;
#pragma unroll
    for (int j = 0; j < NC; j++) {
        const int n = ncol0 + j;
        if (n < N) Dout[((size_t)m * N + n) * nb + b] = (int)__uint_as_float(d[j]);   // an exact integer
    }
}


template <typename ST, bool DUMP>
__global__ void __launch_bounds__(THREADS, 1) gemm_w4a8_tcf_kernel(
    const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
    const float *__restrict__ xs, const ST *__restrict__ sw, float *__restrict__ Y, int32_t *__restrict__ Dout,
    int M, int N, int K, int nsplit, int gsplit) {
    extern __shared__ unsigned char smem_dyn[];
    const uint32_t raw = ptx::smem_u32(smem_dyn);
    const uint32_t base = (raw + 1023u) & ~1023u;
    unsigned char *base_ptr = smem_dyn + (base - raw);
    const uint32_t bar0 = base + OFF_BAR;
    auto BAR = [&](int idx) { return bar0 + 8u * idx; };
    constexpr int AR_FULL = 0, AR_EMPTY = AR_FULL + SR, BR_FULL = AR_EMPTY + SR, BR_EMPTY = BR_FULL + SR,
                  OP_FULL = BR_EMPTY + SR, OP_EMPTY = OP_FULL + SO, SW_FULL = OP_EMPTY + SO, SW_EMPTY = SW_FULL + SS,
                  TM_FULL = SW_EMPTY + SS, TM_EMPTY = TM_FULL + TB;
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(base_ptr + OFF_TMEM);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nb = K / QBLK;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const int num_tiles = m_tiles * n_tiles;
    const int num_work = num_tiles * nsplit;

    if (tid == 0) {
        for (int i = 0; i < SR; i++) {
            ptx::mbar_init(BAR(AR_FULL + i), 1); ptx::mbar_init(BAR(AR_EMPTY + i), CONV_WARPS);
            ptx::mbar_init(BAR(BR_FULL + i), 1); ptx::mbar_init(BAR(BR_EMPTY + i), CONV_WARPS);
        }
        for (int i = 0; i < SO; i++) { ptx::mbar_init(BAR(OP_FULL + i), CONV_WARPS); ptx::mbar_init(BAR(OP_EMPTY + i), 1); }
        for (int i = 0; i < SS; i++) { ptx::mbar_init(BAR(SW_FULL + i), CONV_WARPS); ptx::mbar_init(BAR(SW_EMPTY + i), EPI_WARPS); }
        for (int i = 0; i < TB; i++) { ptx::mbar_init(BAR(TM_FULL + i), 1); ptx::mbar_init(BAR(TM_EMPTY + i), EPI_WARPS); }
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
            Ring ra(SR), rb(SR);
            bool ok = true;
            for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
                const Work wk = decode_work<false>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gemm::GroupList());
                for (int kt = 0; kt < wk.nkt && ok; kt++) {
                    const int kel = (wk.g0 + kt * GPK) * QBLK;
                    if (!ptx::mbar_wait(BAR(AR_EMPTY + ra.stage), ra.phase ^ 1u)) { dev_set_error(gemm::ERR_PRODUCER | 1); ok = false; break; }
                    ptx::mbar_arrive_expect_tx(BAR(AR_FULL + ra.stage), ARAW);
                    ptx::tma_load_2d(base + OFF_ARAW + ra.stage * ARAW, &tmA, kel, wk.m0, BAR(AR_FULL + ra.stage));
                    ra.advance();
                    if (!ptx::mbar_wait(BAR(BR_EMPTY + rb.stage), rb.phase ^ 1u)) { dev_set_error(gemm::ERR_PRODUCER | 2); ok = false; break; }
                    ptx::mbar_arrive_expect_tx(BAR(BR_FULL + rb.stage), BRAW);
                    ptx::tma_load_2d(base + OFF_BRAW + rb.stage * BRAW, &tmB, kel / 2, wk.n0, BAR(BR_FULL + rb.stage));
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
            Ring ro(SO), rt(TB);
            const uint32_t idesc = umma_idesc_f16(BM, BN);
            bool ok = true;
            for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
                const Work wk = decode_work<false>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gemm::GroupList());
                for (int kt = 0; kt < wk.nkt && ok; kt++) {
                    if (!ptx::mbar_wait(BAR(OP_FULL + ro.stage), ro.phase)) { dev_set_error(gemm::ERR_MMA | 1); ok = false; break; }
                    ptx::tc_fence_after_sync();
                    const uint64_t adesc = ptx::umma_desc_k_sw128(base + OFF_OPA + ro.stage * OPA);
                    const uint64_t bdesc = ptx::umma_desc_k_sw128(base + OFF_OPB + ro.stage * OPB);
                    const int ng = min(GPK, wk.g1 - (wk.g0 + kt * GPK));
                    for (int g = 0; g < ng; g++) {
                        if (!ptx::mbar_wait(BAR(TM_EMPTY + rt.stage), rt.phase ^ 1u)) { dev_set_error(gemm::ERR_MMA | 3); ok = false; break; }
                        ptx::tc_fence_after_sync();
                        // group g = 64 bytes at offset (g % 2) * 64 of every row of swizzle atom g / 2; two K = 16 MMAs
                        const uint64_t off = (uint64_t)(((g >> 1) * ATOM + (g & 1) * 64) >> 4);
                        umma_f16(tmem_base + rt.stage * BN, adesc + off, bdesc + off, idesc, 0u);
                        umma_f16(tmem_base + rt.stage * BN, adesc + off + 2, bdesc + off + 2, idesc, 1u);
                        ptx::umma_commit(BAR(TM_FULL + rt.stage));
                        rt.advance();
                    }
                    ptx::umma_commit(BAR(OP_EMPTY + ro.stage));
                    ro.advance();
                }
            }
        }
    } else if (warp < 2 + CONV_WARPS) {
        // ---------------- integer -> fp16 conversion of both operands + weight-scale staging ----------------
        const int ct = tid - 64;  // 0..CONV_WARPS*32-1
        Ring ra(SR), rb(SR), ro(SO), rs(SS);
        bool ok = true;
        for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
            const Work wk = decode_work<false>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gemm::GroupList());
            const int n0 = wk.n0;
            for (int kt = 0; kt < wk.nkt && ok; kt++) {
                bool w = ptx::mbar_wait_warp(BAR(AR_FULL + ra.stage), ra.phase) && ptx::mbar_wait_warp(BAR(BR_FULL + rb.stage), rb.phase) &&
                         ptx::mbar_wait_warp(BAR(OP_EMPTY + ro.stage), ro.phase ^ 1u);
                if (!w) { dev_set_error(gemm::ERR_DEQUANT | 1); ok = false; break; }
                const unsigned char *asrc = base_ptr + OFF_ARAW + ra.stage * ARAW;
                const unsigned char *bsrc = base_ptr + OFF_BRAW + rb.stage * BRAW;
                unsigned char *adst = base_ptr + OFF_OPA + ro.stage * OPA;
                unsigned char *bdst = base_ptr + OFF_OPB + ro.stage * OPB;
#pragma unroll
                for (int i = 0; i < (BM * 8) / (CONV_WARPS * 32); i++) {
                    const int j = ct + i * CONV_WARPS * 32;
                    const int r = j >> 3, c = j & 7;      // row r, 16 int8 = elements [16c, 16c+16) -> output chunks 2c, 2c+1
                    const uint4 v = *reinterpret_cast<const uint4 *>(asrc + r * KT + c * 16);
                    *reinterpret_cast<uint4 *>(adst + op_chunk(r, 2 * c)) = i8_to_f16x8(v.x, v.y);
                    *reinterpret_cast<uint4 *>(adst + op_chunk(r, 2 * c + 1)) = i8_to_f16x8(v.z, v.w);
                }
#pragma unroll
                for (int i = 0; i < (BN * 8) / (CONV_WARPS * 32); i++) {
                    const int j = ct + i * CONV_WARPS * 32;
                    const int n = j >> 3, c = j & 7;      // row n, 8 packed bytes = elements [16c, 16c+16)
                    const uint2 p = *reinterpret_cast<const uint2 *>(bsrc + n * (KT / 2) + c * 8);
                    *reinterpret_cast<uint4 *>(bdst + op_chunk(n, 2 * c)) = w4_to_f16x8(p.x);
                    *reinterpret_cast<uint4 *>(bdst + op_chunk(n, 2 * c + 1)) = w4_to_f16x8(p.y);
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(BAR(OP_FULL + ro.stage));
                    ptx::mbar_arrive(BAR(AR_EMPTY + ra.stage));
                    ptx::mbar_arrive(BAR(BR_EMPTY + rb.stage));
                }
                ra.advance(); rb.advance(); ro.advance();

                w = ptx::mbar_wait_warp(BAR(SW_EMPTY + rs.stage), rs.phase ^ 1u);
                if (!w) { dev_set_error(gemm::ERR_DEQUANT | 2); ok = false; break; }
                float *ssw = reinterpret_cast<float *>(base_ptr + OFF_SW + rs.stage * SW_STAGE);
                {
                    const int nl = ct, n = n0 + nl;       // CONV_WARPS * 32 == BN: one weight row per thread
#pragma unroll
                    for (int g = 0; g < GPK; g++) {
                        const int b = wk.g0 + kt * GPK + g;
                        float v = 0.f;
                        if (!DUMP && n < N && b < wk.g1) v = sval(sw[(size_t)n * nb + b]);
                        ssw[g * BN + nl] = v;
                    }
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(BAR(SW_FULL + rs.stage));
                rs.advance();
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int ew = warp - (2 + CONV_WARPS);
        const int quad = warp & 3;              // TMEM lanes [32*quad, 32*quad+32)
        const int col0 = (ew >> 2) * EPI_COLS;
        Ring rs(SS), rt(TB);
        bool ok = true;
        for (int wi = blockIdx.x; wi < num_work && ok; wi += gridDim.x) {
            const Work wk = decode_work<false>(wi, m_tiles, num_tiles, nb, gsplit, M, N, n_tiles, gemm::GroupList());
            const int m0 = wk.m0, n0 = wk.n0;
            const int m = m0 + quad * 32 + lane;
            const bool rows_live = (m0 + quad * 32) < M;
            const float *xsrow = xs + (size_t)(m < M ? m : 0) * nb;
            float acc[EPI_COLS];
#pragma unroll
            for (int j = 0; j < EPI_COLS; j++) acc[j] = 0.f;
            float xnext[GPK];
#pragma unroll
            for (int g = 0; g < GPK; g++) xnext[g] = (!DUMP && m < M && wk.g0 + g < wk.g1) ? xsrow[wk.g0 + g] : 0.f;
            for (int kt = 0; kt < wk.nkt && ok; kt++) {
                float xcur[GPK];
#pragma unroll
                for (int g = 0; g < GPK; g++) {
                    xcur[g] = xnext[g];
                    const int b = wk.g0 + (kt + 1) * GPK + g;
                    xnext[g] = (!DUMP && m < M && b < wk.g1) ? xsrow[b] : 0.f;
                }
                const int ng = min(GPK, wk.g1 - (wk.g0 + kt * GPK));
                const uint32_t tlane = tmem_base + ((uint32_t)(quad * 32) << 16) + col0;
                // chunks of EPI_CH columns, software-pipelined: chunk i+1 is in flight while chunk i is processed
                uint32_t d0[EPI_CH], d1[EPI_CH];
                bool w = ptx::mbar_wait_warp(BAR(TM_FULL + rt.stage), rt.phase);
                if (!w) { dev_set_error(gemm::ERR_EPILOGUE | 2); ok = false; break; }
                ptx::tc_fence_after_sync();
                if (rows_live) ptx::tmem_ld(tlane + rt.stage * BN, d0);
                w = ptx::mbar_wait_warp(BAR(SW_FULL + rs.stage), rs.phase);
                if (!w) { dev_set_error(gemm::ERR_EPILOGUE | 1); ok = false; break; }
                const float *ssw = reinterpret_cast<const float *>(base_ptr + OFF_SW + rs.stage * SW_STAGE) + col0;
#pragma unroll
                for (int g = 0; g < GPK; g++) {
                    if (g < ng) {
                        const int b = wk.g0 + kt * GPK + g;
                        const uint32_t tcur = tlane + rt.stage * BN;
#pragma unroll
                        for (int c = 0; c < EPI_COLS / EPI_CH; c += 2) {
                            // even chunk c lives in d0, odd chunk c+1 in d1
                            ptx::tmem_ld_wait();
                            if (rows_live) ptx::tmem_ld(tcur + (c + 1) * EPI_CH, d1);
                            if (rows_live) {
                                if (DUMP) epi_dump_f<EPI_CH>(d0, Dout, m, M, n0 + col0 + c * EPI_CH, N, nb, b);
                                else epi_chunk_f<EPI_CH>(d0, xcur[g], ssw + g * BN + c * EPI_CH, acc + c * EPI_CH);
                            }
                            ptx::tmem_ld_wait();
                            const bool last = (c + 2 >= EPI_COLS / EPI_CH);
                            if (!last) {
                                if (rows_live) ptx::tmem_ld(tcur + (c + 2) * EPI_CH, d0);
                            } else {
                                // all of this warp's columns of the group are in registers: release the buffer,
                                // then start on the next group's first chunk
                                ptx::tc_fence_before_sync();
                                __syncwarp();
                                if (lane == 0) ptx::mbar_arrive(BAR(TM_EMPTY + rt.stage));
                                rt.advance();
                                if (g + 1 < ng) {
                                    w = ptx::mbar_wait_warp(BAR(TM_FULL + rt.stage), rt.phase);
                                    if (!w) { dev_set_error(gemm::ERR_EPILOGUE | 3); ok = false; }
                                    ptx::tc_fence_after_sync();
                                    if (ok && rows_live) ptx::tmem_ld(tlane + rt.stage * BN, d0);
                                }
                            }
                            if (rows_live) {
                                if (DUMP) epi_dump_f<EPI_CH>(d1, Dout, m, M, n0 + col0 + (c + 1) * EPI_CH, N, nb, b);
                                else epi_chunk_f<EPI_CH>(d1, xcur[g], ssw + g * BN + (c + 1) * EPI_CH, acc + (c + 1) * EPI_CH);
                            }
                        }
                        if (!ok) break;
                    }
                }
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(BAR(SW_EMPTY + rs.stage));
                rs.advance();
            }
            if (!DUMP && ok && m < M) {
                float *yrow = Y + (size_t)wk.split * ((size_t)M * N) + (size_t)m * N + n0 + col0;
                const int nleft = N - (n0 + col0);
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

    // ---------------- teardown ----------------
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, TB * BN);
    }
}

// ---- host side ------------------------------------------------------------------------------------------------
template <typename ST, bool DUMP>
inline int launch_t(const int8_t *X, const float *xs, const uint8_t *Wq, const ST *sw, float *Y, int32_t *D,
                    int M, int N, int K, int nsplit, int gsplit, cudaStream_t st) {
    CUtensorMap tmA, tmB;
    int rc = make_tmap_u8(&tmA, X, (uint64_t)K, (uint64_t)M, KT, BM, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != W4A8_OK) return rc;
    rc = make_tmap_u8(&tmB, Wq, (uint64_t)K / 2, (uint64_t)N, KT / 2, BN, CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != W4A8_OK) return rc;
    auto kern = gemm_w4a8_tcf_kernel<ST, DUMP>;
    static PerDevice<bool> configured_dev;              // the opt-in is a per-device function attribute
    bool &configured = configured_dev.get();
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return cuda_fail(e, "gemm (fp16 operands) smem opt-in");
        configured = true;
    }
    const long tiles = (long)((M + BM - 1) / BM) * ((N + BN - 1) / BN) * nsplit;
    const int sms = sm_count();
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    kern<<<grid, THREADS, SMEM_BYTES, st>>>(tmA, tmB, xs, sw, Y, D, M, N, K, nsplit, gsplit);
    return launch_status("gemm_w4a8_tcf");
}

inline int launch(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y, int M, int N, int K,
                  int scale_dtype, int nsplit, int gsplit, cudaStream_t st) {
    if (scale_dtype == 1)
        return launch_t<__half, false>(X, xs, Wq, (const __half *)sw, Y, nullptr, M, N, K, nsplit, gsplit, st);
    return launch_t<float, false>(X, xs, Wq, (const float *)sw, Y, nullptr, M, N, K, nsplit, gsplit, st);
}
inline int launch_dump(const int8_t *X, const uint8_t *Wq, int32_t *D, int M, int N, int K, cudaStream_t st) {
    return launch_t<float, true>(X, nullptr, Wq, (const float *)nullptr, nullptr, D, M, N, K, 1, K / QBLK, st);
}

}  // namespace gemmf
}  // namespace w4a8
