/*
 * CPU restatement of the dgx-serving W4A8 hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the parity tests, the smoke check and the benchmark's
 * cpu_baseline leg compare against.  Nothing in the shipped library links, loads
 * or calls it; the library has no CPU path at all.
 *
 * Every function restates one piece of the reference (hyunlord/dgx-serving) and
 * names the file:line it follows.  All fp32 arithmetic is IEEE round-to-nearest
 * with explicit fmaf where the reference's nvcc build contracts a*b+c; build with
 * -ffp-contract=off so nothing else is fused.
 *
 * Parity pin: the restatement is checked (tests/test_oracle_pins.py) against
 *   - the LCG-seeded in-test goldens of tests/test_w4a8.cu and tests/test_mma_b1.cu
 *     (regenerated here from their seeds, gates of those tests applied),
 *   - byte fixtures of the on-disk int4 format produced by importing the reference's
 *     tools/extract_weights.py (tests/golden/),
 *   - and, on a GPU box, bit-for-bit against the reference's own kernels rebuilt
 *     for sm_100a (oracle/_ref/libref_kernels.so).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define QBLK 32 /* runtime/config.h:9-11 */

#define API __attribute__((visibility("default")))

/* ---- helpers ---------------------------------------------------------------------------- */

/* IEEE binary16 -> binary32, the value __half2float returns (kernels/qscale.cuh:6). */
static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal half -> normal float */
            int e = -1;
            do { man <<= 1; e++; } while (!(man & 0x400u));
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Weight scale read: float, or __half widened to float (kernels/qscale.cuh:5-6). */
static inline float sval(const void *sw, size_t i, int scale_dtype) {
    if (scale_dtype == 1) return half_to_float(((const uint16_t *)sw)[i]);
    return ((const float *)sw)[i];
}

/* One int4 weight: low nibble = even k, high nibble = odd k, value = nibble - 8
 * (kernels/gemv_w4a8.cuh:16-21, tests/test_w4a8.cu:48-49). */
static inline int wval(const uint8_t *row, int k) {
    uint8_t by = row[k >> 1];
    return (int)((k & 1) ? (by >> 4) : (by & 0x0F)) - 8;
}

API int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

API void oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* LCG of the reference's unit tests (tests/test_w4a8.cu:16): returns a float in [-1, 1). */
API float oracle_lcg_frand(uint32_t *s) {
    *s = *s * 1664525u + 1013904223u;
    return (float)((*s >> 8) & 0xFFFFFFu) / 8388608.0f - 1.0f;
}

API void oracle_lcg_fill(float *dst, size_t n, float mul, uint32_t *s) {
    for (size_t i = 0; i < n; i++) dst[i] = oracle_lcg_frand(s) * mul;
}

/* ---- a1: activation quantization (kernels/quantize_x.cuh:22-39) --------------------------- */
/* X[S,IN] f32 -> xq[S,IN] i8, xs[S,IN/32] f32 (= amax/127), xsum[S,IN/32] i32 (= sum of q). */
API void oracle_quantize_x_q8(const float *X, int8_t *xq, float *xs, int32_t *xsum, int IN, int S) {
    const int nb = IN / QBLK;
#pragma omp parallel for schedule(static)
    for (long gb = 0; gb < (long)S * nb; gb++) {
        const float *x = X + gb * QBLK; /* block gb of row gb/nb: rows are contiguous */
        float amax = 0.0f;
        for (int i = 0; i < QBLK; i++) amax = fmaxf(amax, fabsf(x[i]));
        float d = amax / 127.0f;
        int sum = 0;
        for (int i = 0; i < QBLK; i++) {
            int q = (amax == 0.0f) ? 0 : (int)rintf(x[i] / d);
            q = q < -127 ? -127 : (q > 127 ? 127 : q);
            xq[gb * QBLK + i] = (int8_t)q;
            sum += q;
        }
        xs[gb] = d;
        if (xsum) xsum[gb] = sum;
    }
}

/* ---- producers of quantize_x in the graphs (for the fused entry points) ------------------------------
 * RMSNorm in the order of kernels/rmsnorm.cuh:8-20 + kernels/reduce.cuh:6-24: 256 threads, thread t adds the
 * squares of elements t, t+256, ... (fused multiply-add), a shfl_down tree per warp of 32 threads, then one
 * more tree over the 8 warp sums; inv = 1/sqrt(ss/hh + eps).  The GPU uses its reciprocal-square-root
 * approximation (rsqrtf), so this restatement is close (a few ulp), not bit-equal: the bitwise proof of the
 * fused kernels is against the reference's own kernels on the GPU.  variant 0: y = x*inv*W, 1: y = x*inv*(1+W),
 * 2: y = x*inv. */
static float tree32(float *v) { /* lane 0's value after shfl_down by 16, 8, 4, 2, 1 (lanes past the end keep their own value) */
    for (int o = 16; o > 0; o >>= 1)
        for (int l = 0; l < 32; l++) v[l] = v[l] + (l + o < 32 ? v[l + o] : v[l]);
    return v[0];
}
API void oracle_rmsnorm(const float *X, const float *W, float *Y, int rows, int hh, float eps, int variant) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; r++) {
        const float *x = X + (size_t)r * hh;
        float part[256], ws[32];
        for (int t = 0; t < 256; t++) {
            float ss = 0.0f;
            for (int i = t; i < hh; i += 256) ss = fmaf(x[i], x[i], ss);
            part[t] = ss;
        }
        for (int w = 0; w < 32; w++) ws[w] = 0.0f;
        for (int w = 0; w < 8; w++) ws[w] = tree32(part + 32 * w);
        const float ss = tree32(ws);
        const float inv = 1.0f / sqrtf(ss / (float)hh + eps);
        for (int i = 0; i < hh; i++) {
            const float xi = x[i] * inv;
            Y[(size_t)r * hh + i] = variant == 0 ? xi * W[i] : (variant == 1 ? xi * (1.0f + W[i]) : xi);
        }
    }
}
/* SwiGLU (act 0, kernels/swiglu.cuh:5-8) and GeGLU (act 1, :19-27); the C library's expf / tanhf stand for the GPU's. */
API void oracle_glu(const float *g, const float *u, float *Y, long n, int act) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < n; i++) {
        const float x = g[i];
        if (act == 0) { const float s = x / (1.0f + expf(-x)); Y[i] = s * u[i]; }
        else { const float t = tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)); Y[i] = 0.5f * x * (1.0f + t) * u[i]; }
    }
}

/* ---- weight producers ----------------------------------------------------------------------- */
/* Round-to-nearest int4 packer.  zero_scale = 1.0f restates tests/test_w4a8.cu:19-27
 * (lrintf = round half to even); zero_scale = 1e-8f restates tools/extract_weights.py:124-140
 * (np.round is also half to even). */
API void oracle_pack_q4(const float *W, int OUT, int IN, uint8_t *Wq, float *sc, float zero_scale) {
    const int nb = IN / QBLK;
    memset(Wq, 0, (size_t)OUT * (IN / 2));
#pragma omp parallel for schedule(static)
    for (int o = 0; o < OUT; o++) {
        for (int b = 0; b < nb; b++) {
            const float *w = W + (size_t)o * IN + (size_t)b * QBLK;
            float mx = 0.0f;
            for (int i = 0; i < QBLK; i++) mx = fmaxf(mx, fabsf(w[i]));
            float s = mx / 7.0f;
            if (s == 0.0f) s = zero_scale;
            sc[(size_t)o * nb + b] = s;
            for (int i = 0; i < QBLK; i++) {
                int n = b * QBLK + i;
                int q = (int)lrintf(w[i] / s) + 8;
                if (q < 0) q = 0;
                if (q > 15) q = 15;
                uint8_t *by = &Wq[(size_t)o * (IN / 2) + (n >> 1)];
                if (n & 1) *by = (uint8_t)((*by & 0x0F) | (q << 4));
                else *by = (uint8_t)((*by & 0xF0) | q);
            }
        }
    }
}

/* ---- A3: exact integer group dots D[m,n,b] (tests/test_mma_b1.cu:52-58) ------------------- */
API void oracle_group_dots(const int8_t *xq, const uint8_t *Wq, int32_t *D, int M, int N, int K) {
    const int nb = K / QBLK;
#pragma omp parallel for schedule(static)
    for (long mn = 0; mn < (long)M * N; mn++) {
        int m = (int)(mn / N), n = (int)(mn % N);
        const int8_t *x = xq + (size_t)m * K;
        const uint8_t *w = Wq + (size_t)n * (K / 2);
        for (int b = 0; b < nb; b++) {
            int dot = 0;
            for (int i = 0; i < QBLK; i++) {
                int k = b * QBLK + i;
                dot += (int)x[k] * wval(w, k);
            }
            D[(size_t)mn * nb + b] = dot;
        }
    }
}

/* ---- fp64 golden (tests/test_w4a8.cu:44-56) ------------------------------------------------- */
API void oracle_w4a8_f64(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw,
                         double *Y, int M, int N, int K, int scale_dtype) {
    const int nb = K / QBLK;
#pragma omp parallel for schedule(static)
    for (long mn = 0; mn < (long)M * N; mn++) {
        int m = (int)(mn / N), n = (int)(mn % N);
        const int8_t *x = xq + (size_t)m * K;
        const uint8_t *w = Wq + (size_t)n * (K / 2);
        double acc = 0.0;
        for (int b = 0; b < nb; b++) {
            double dot = 0.0;
            float dx = xs[(size_t)m * nb + b];
            float s = sval(sw, (size_t)n * nb + b, scale_dtype);
            for (int i = 0; i < QBLK; i++) {
                int k = b * QBLK + i;
                double wv = (double)wval(w, k) * (double)s;
                dot += (double)x[k] * (double)dx * wv;
            }
            acc += dot;
        }
        Y[mn] = acc;
    }
}

/* ---- a4-a8: GEMV family, fp32 in the reference's evaluation order ------------------------- */
/* kernels/gemv_w4a8.cuh:37-48: lane l visits the 8-element chunks base = 8l + 256i in
 * increasing i; per chunk an int32 dot over 8 elements, then acc = fma(xs*sw, (float)dot, acc);
 * kernels/reduce.cuh:6-9: shfl_down tree 16,8,4,2,1, lane 0 holds the result.  The mlp, SB, g4
 * and gemm_batch variants keep this order per row (kernels/gemv_w4a8.cuh:51-53,118,182-190;
 * kernels/gemm_batch.cuh:199-211). */
API void oracle_gemv_w4a8(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw,
                          float *Y, int IN, int OUT, int S, int scale_dtype) {
    const int nb = IN / QBLK;
#pragma omp parallel for schedule(static)
    for (long so = 0; so < (long)S * OUT; so++) {
        int s = (int)(so / OUT), o = (int)(so % OUT);
        const int8_t *x = xq + (size_t)s * IN;
        const uint8_t *w = Wq + (size_t)o * (IN / 2);
        float lane_acc[32];
        for (int lane = 0; lane < 32; lane++) {
            float acc = 0.0f;
            for (int base = lane * 8; base < IN; base += 256) {
                int blk = base / QBLK;
                float sc_b = xs[(size_t)s * nb + blk] * sval(sw, (size_t)o * nb + blk, scale_dtype);
                int dot = 0;
                for (int i = 0; i < 8; i++) dot += (int)x[base + i] * wval(w, base + i);
                acc = fmaf(sc_b, (float)dot, acc);
            }
            lane_acc[lane] = acc;
        }
        for (int off = 16; off > 0; off >>= 1) {
            float nxt[32];
            for (int lane = 0; lane < 32; lane++)
                nxt[lane] = lane_acc[lane] + ((lane + off < 32) ? lane_acc[lane + off] : lane_acc[lane]);
            memcpy(lane_acc, nxt, sizeof(nxt));
        }
        Y[so] = lane_acc[0];
    }
}

/* The B200 library's own GEMV-family order (it reads one whole group per lane with 128-bit loads, so
 * the reference's per-8-element chain does not apply): chain c = b mod 32 accumulates
 * acc_c = fma(xs*sw, (float)D_b, acc_c) over b = c, c+32, ... ascending, D_b the full 32-element group
 * dot; then the same shfl_down tree as kernels/reduce.cuh:6-9.  Used for bit-exact checks of the CUDA
 * GEMV; it is a restatement of the library's documented order, not of the reference. */
API void oracle_gemv_b200_order(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw,
                                float *Y, int IN, int OUT, int S, int scale_dtype) {
    const int nb = IN / QBLK;
#pragma omp parallel for schedule(static)
    for (long so = 0; so < (long)S * OUT; so++) {
        int s = (int)(so / OUT), o = (int)(so % OUT);
        const int8_t *x = xq + (size_t)s * IN;
        const uint8_t *w = Wq + (size_t)o * (IN / 2);
        float lane_acc[32];
        for (int lane = 0; lane < 32; lane++) {
            float acc = 0.0f;
            for (int b = lane; b < nb; b += 32) {
                float sc_b = xs[(size_t)s * nb + b] * sval(sw, (size_t)o * nb + b, scale_dtype);
                int dot = 0;
                for (int i = 0; i < QBLK; i++) dot += (int)x[b * QBLK + i] * wval(w, b * QBLK + i);
                acc = fmaf(sc_b, (float)dot, acc);
            }
            lane_acc[lane] = acc;
        }
        for (int off = 16; off > 0; off >>= 1) {
            float nxt[32];
            for (int lane = 0; lane < 32; lane++)
                nxt[lane] = lane_acc[lane] + ((lane + off < 32) ? lane_acc[lane + off] : lane_acc[lane]);
            memcpy(lane_acc, nxt, sizeof(nxt));
        }
        Y[so] = lane_acc[0];
    }
}

/* ---- a9-a12: MMQ / MMA family, fp32 in the reference's evaluation order ------------------- */
/* kernels/gemm_mmq.cuh:77,98-106 (and gemm_mma.cuh:100-103): for group b ascending,
 * t = (float)D * xs[m,b] (rounded), acc = fma(t, sw[n,b], acc).  Tile shape, raster order and
 * pipeline depth do not enter (kernels/gemm_mmq_tmpl.cuh:106-109, gemm_mmq_raster.cuh:6). */
API void oracle_gemm_mmq_w4a8(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw,
                              float *Y, int M, int N, int K, int scale_dtype) {
    const int nb = K / QBLK;
#pragma omp parallel for schedule(static)
    for (long mn = 0; mn < (long)M * N; mn++) {
        int m = (int)(mn / N), n = (int)(mn % N);
        const int8_t *x = X + (size_t)m * K;
        const uint8_t *w = Wq + (size_t)n * (K / 2);
        float acc = 0.0f;
        for (int b = 0; b < nb; b++) {
            int dot = 0;
            for (int i = 0; i < QBLK; i++) {
                int k = b * QBLK + i;
                dot += (int)x[k] * wval(w, k);
            }
            float t = (float)dot * xs[(size_t)m * nb + b];
            acc = fmaf(t, sval(sw, (size_t)n * nb + b, scale_dtype), acc);
        }
        Y[mn] = acc;
    }
}

/* a13: BM=16 split-K (kernels/gemm_mmq.cuh:128-219): K-tiles of 64 split into `splitk`
 * contiguous ranges of ceil(niter/splitk) tiles, each summed in MMQ order, partials added in
 * ascending split order starting from 0.0f (kernels/gemm_mmq.cuh:201-204). */
API void oracle_gemm_splitk_w4a8(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw,
                                 float *Y, int M, int N, int K, int scale_dtype, int splitk) {
    const int nb = K / QBLK;
    const int KS = 2; /* KT=64 -> 2 groups per K-tile */
    const int niter = (nb + KS - 1) / KS;
    const int itper = (niter + splitk - 1) / splitk;
#pragma omp parallel for schedule(static)
    for (long mn = 0; mn < (long)M * N; mn++) {
        int m = (int)(mn / N), n = (int)(mn % N);
        const int8_t *x = X + (size_t)m * K;
        const uint8_t *w = Wq + (size_t)n * (K / 2);
        float total = 0.0f;
        for (int sp = 0; sp < splitk; sp++) {
            int it0 = sp * itper, it1 = (sp + 1) * itper < niter ? (sp + 1) * itper : niter;
            float acc = 0.0f;
            for (int b = it0 * KS; b < it1 * KS && b < nb; b++) {
                int dot = 0;
                for (int i = 0; i < QBLK; i++) {
                    int k = b * QBLK + i;
                    dot += (int)x[k] * wval(w, k);
                }
                float t = (float)dot * xs[(size_t)m * nb + b];
                acc = fmaf(t, sval(sw, (size_t)n * nb + b, scale_dtype), acc);
            }
            total = (splitk == 1) ? acc : total + acc;
        }
        Y[mn] = total;
    }
}

/* Sum over groups of |D * xs * sw| per output: the normaliser of the per-element gate in
 * tests/gemma4_mmq/shape.cu:105-117. */
API void oracle_abs_terms(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw,
                          double *T, int M, int N, int K, int scale_dtype) {
    const int nb = K / QBLK;
#pragma omp parallel for schedule(static)
    for (long mn = 0; mn < (long)M * N; mn++) {
        int m = (int)(mn / N), n = (int)(mn % N);
        const int8_t *x = X + (size_t)m * K;
        const uint8_t *w = Wq + (size_t)n * (K / 2);
        double acc = 0.0;
        for (int b = 0; b < nb; b++) {
            int dot = 0;
            for (int i = 0; i < QBLK; i++) {
                int k = b * QBLK + i;
                dot += (int)x[k] * wval(w, k);
            }
            acc += fabs((double)dot * (double)xs[(size_t)m * nb + b] *
                        (double)sval(sw, (size_t)n * nb + b, scale_dtype));
        }
        T[mn] = acc;
    }
}

/* ---- grouped experts (W4A8 semantics applied per expert slice) ---------------------------- */
/* The reference's expert kernels are W4A32 (kernels/moe_fused.cuh:14-33); what is kept from them
 * is the indexing: expert e's weights start e*(OUT*IN/2) bytes into the flat tensor and its scales
 * e*(OUT*IN/32) elements in (kernels/moe_fused.cuh:21-24), slot = token*topk + k, expert id
 * idx[slot].  Each slot's row is one dense W4A8 product in MMQ order against its expert.
 * xq/xs are per slot when x_per_slot != 0 (down projection), else per token (gate/up). */
API void oracle_moe_w4a8(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw,
                         const int32_t *idx, float *Y, int nslots, int topk, int x_per_slot,
                         int N, int K, int scale_dtype) {
    const int nb = K / QBLK;
#pragma omp parallel for schedule(static)
    for (long sn = 0; sn < (long)nslots * N; sn++) {
        int slot = (int)(sn / N), n = (int)(sn % N);
        int e = idx[slot];
        int row = x_per_slot ? slot : slot / topk;
        const int8_t *x = xq + (size_t)row * K;
        const uint8_t *w = Wq + (size_t)e * ((size_t)N * K / 2) + (size_t)n * (K / 2);
        size_t sbase = (size_t)e * ((size_t)N * nb) + (size_t)n * nb;
        float acc = 0.0f;
        for (int b = 0; b < nb; b++) {
            int dot = 0;
            for (int i = 0; i < QBLK; i++) {
                int k = b * QBLK + i;
                dot += (int)x[k] * wval(w, k);
            }
            float t = (float)dot * xs[(size_t)row * nb + b];
            acc = fmaf(t, sval(sw, sbase + b, scale_dtype), acc);
        }
        Y[sn] = acc;
    }
}

/* Combine of the routed-expert block: out[b][o] = sum over k ascending, from 0, of dw[b*topk+k] * so[b*topk+k][o],
 * the product rounded to fp32 before it is added: the values of kernels/moe_fused.cuh:64 (Sout = dw * acc) summed in
 * the fixed order of kernels/moe_fused.cuh:68-76.  Built with -ffp-contract=off, so no fused multiply-add. */
API void oracle_moe_combine(const float *so, const float *dw, float *out, int S, int topk, int H) {
#pragma omp parallel for schedule(static)
    for (long i = 0; i < (long)S * H; i++) {
        long b = i / H;
        int o = (int)(i % H);
        float acc = 0.0f;
        for (int k = 0; k < topk; k++) {
            long slot = b * topk + k;
            float t = dw[slot] * so[slot * H + o];
            acc = acc + t;
        }
        out[i] = acc;
    }
}
