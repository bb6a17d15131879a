/*
 * w4a8_b200 — C ABI of the B200 (sm_100a) W4A8 quantized-matmul library.
 *
 * Drop-in replacement for the header-only `launch_*` kernel launchers of hyunlord/dgx-serving's
 * W4A8 path (kernels/quantize_x.cuh, gemv_w4a8.cuh, gemm_batch.cuh, gemm_mma.cuh, gemm_mmq*.cuh)
 * and for the whole-file weight upload of runtime/weights*.cu.  Each entry point cites the
 * reference interface it replaces.  Same-named C++ shim launchers that forward to this ABI live in
 * dgx-serving_b200/kernels/.
 *
 * Conventions (they mirror the reference's):
 *   - Every pointer is a DEVICE pointer owned by the caller unless the name says `host`.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the default stream).  Launch entry points
 *     only enqueue work: no synchronisation, no allocation, no host-side branching on device data,
 *     so they may be called under CUDA-graph stream capture like the reference launchers
 *     (models/gemma4_decode.cu:180-189).
 *   - Data formats are the reference's: Wq[N][K/2] uint8, byte j of a row = element 2j in the low
 *     nibble and 2j+1 in the high nibble, value = nibble - 8 (kernels/gemv_w4a8.cuh:16-21);
 *     sw[N][K/32] per-group scales, fp32 (scale_dtype 0) or fp16 (scale_dtype 1)
 *     (runtime/config.h:44-45); xq[S][K] int8 with xs[S][K/32] fp32 per-32-block scales
 *     (kernels/quantize_x.cuh:6-11).  K must be a multiple of 32.
 *   - The reference launchers return void and never check errors (callers synchronise and exit on
 *     any CUDA error, models/qwen35_decode.cu:24-25,229).  These return an int status instead:
 *     0 on success, a W4A8_ERR_* code otherwise, with w4a8_last_error() giving the text.  There is
 *     no CPU fallback: without a usable sm_100 device every launch entry point fails.
 *   - One host thread at a time inside the library, like the reference (one process per GPU is the intended
 *     deployment): the kernel-selection switches of w4a8_config and the launch caches (shared-memory opt-in and
 *     occupancy per device, tensor maps) are plain process-wide state without locks.  One thread may drive several
 *     devices (the caches are keyed by the current device); concurrent calls from several threads are not supported.
 */
#ifndef W4A8_B200_H
#define W4A8_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define W4A8_QBLK 32 /* runtime/config.h:9-11 */

enum {
    W4A8_OK = 0,
    W4A8_ERR_ARG = 1,         /* null pointer, K % 32 != 0, negative size, unknown scale_dtype ... */
    W4A8_ERR_ALIGN = 2,       /* a pointer or pitch misses the alignment the entry point documents */
    W4A8_ERR_CUDA = 3,        /* a CUDA runtime / driver call failed (text in w4a8_last_error) */
    W4A8_ERR_IO = 4,          /* weight file missing or shorter than the shape requires */
    W4A8_ERR_DEVICE = 5,      /* a kernel recorded a device-side error (bounded wait ran out) */
    W4A8_ERR_UNSUPPORTED = 6, /* not an sm_100 device, or a size beyond a documented maximum */
    W4A8_ERR_WORKSPACE = 7    /* caller-provided workspace too small */
};

/* Library version (major*10000 + minor*100 + patch). */
int w4a8_version(void);
/* Text of the last failure on this host thread ("" if none). */
const char *w4a8_last_error(void);
/* Reads and clears the device-side error word that kernels with bounded waits set when a wait runs
 * out.  Synchronises the device.  Returns W4A8_OK or W4A8_ERR_DEVICE (detail in *detail if given). */
int w4a8_device_status(uint32_t *detail);

/* Run-time policy switches (the reference keeps such switches in runtime/knobs.h, read from the environment;
 * the same names are read here once: W4A8_GEMV = dp4a | mma | bulk, W4A8_PDL = 0 | 1).
 *   "gemv_kernel": 0 = auto (default): 2..16 activation rows use the tensor-path kernel; one row uses the dp4a
 *                  streaming kernel, or the bulk-copy streaming kernel when the row has 2048..8192 elements and the
 *                  matrix is large (96 MB of weights or more) or its scales are fp16; one row with fp16 scales outside
 *                  that range uses the tensor-path kernel.  1 = dp4a kernel for every S; 2 = tensor-path kernel for
 *                  every S it supports (K % 256 == 0, 16-byte aligned Wq and sw); 3 = bulk-copy kernel for every
 *                  single row it supports (K % 128 == 0, K <= 8192, 16-byte aligned Wq and sw), dp4a otherwise;
 *                  5 = tcgen05 kernel (weights on the MMA's M side, MMQ order) for up to 16 rows per pass where it
 *                  applies (16-byte aligned Wq and sw; slower than the default kernels, kept as a measured alternative).
 *                  The tensor-path kernel evaluates fp32 in the MMQ order (bit-identical to w4a8_gemm and to the
 *                  reference's MMQ kernels); the dp4a and bulk-copy kernels share one fixed order of their own (within
 *                  1e-5).  Policy 2 therefore makes a row's bits independent of S for all S >= 1 (the reference's
 *                  batch == single invariant), policy 0 for all S >= 2.
 *   "gemm_kernel": which tensor-core kernel w4a8_gemm / w4a8_gemm_splitk / w4a8_linear use (environment:
 *                  W4A8_GEMM = i8 | f16).  1 = int8 operands, tcgen05.mma kind::i8, int32 group dots converted in
 *                  the epilogue (default, the faster one); 0 = operands converted to fp16 on the way into shared
 *                  memory (every int4 and int8 value is exact in fp16), tcgen05.mma kind::f16 with fp32
 *                  accumulation of one 32-element group, which is exact as well (|sum| <= 32*127*8 < 2^24).
 *                  Both give the same bits.
 *   "moe_kernel":  w4a8_moe_block's expert products: 0 = by slot count (default), 1 = grouped GEMV, 2 = sorted grouped
 *                  tensor-core GEMM. */
int w4a8_config(const char *key, int value);

/* ---- a1: activation quantization ------------------------------------------------------------------
 * Replaces launch_quantize_x_q8 (kernels/quantize_x.cuh:41-47).
 * X[S,IN] fp32 -> xq[S,IN] int8, xs[S,IN/32] fp32 (= amax/127), xsum[S,IN/32] int32 (= sum of xq over
 * the block; may be NULL).  Bit-exact with the reference: d = amax/127.0f, q = rintf(x/d) clamped to
 * +-127, all-zero block -> q = 0, d = 0. */
int w4a8_quantize_x_q8(const float *X, int8_t *xq, float *xs, int32_t *xsum, int IN, int S, void *stream);

/* ---- quantize_x fused into its producer (the first of the follow-ups after the path itself) ------------------------
 * The reference's graphs run norm -> quantize_x -> matmul and activation -> quantize_x -> down projection as
 * separate kernels (models/qwen35_decode.cu:148-149 and 215-218).  These two entries do producer and quantizer in
 * one kernel and give the SAME xq / xs / xsum, bit for bit, as the reference's two-kernel sequence:
 *   w4a8_rmsnorm_quantize_x_q8 = launch_rmsnorm (variant 0, y = x*inv*W, kernels/rmsnorm.cuh:8-25),
 *     launch_rmsnorm_zc (variant 1, y = x*inv*(1+W), :30-47) or launch_rmsnorm_noscale (variant 2, :50-67)
 *     followed by launch_quantize_x_q8; inv = rsqrtf(mean(x^2) + eps) with the reference's reduction order.
 *   w4a8_glu_quantize_x_q8 = launch_swiglu (act 0, kernels/swiglu.cuh:5-14) or launch_geglu (act 1, :19-33)
 *     followed by launch_quantize_x_q8.
 * Y, if not NULL, also receives the fp32 intermediate [S, IN] (for a consumer that is not quantized).  X, W, G, U, Y
 * must be 16-byte aligned; IN a multiple of 32. */
int w4a8_rmsnorm_quantize_x_q8(const float *X, const float *W, float eps, int variant, float *Y, int8_t *xq,
                               float *xs, int32_t *xsum, int IN, int S, void *stream);
int w4a8_glu_quantize_x_q8(const float *G, const float *U, int act, float *Y, int8_t *xq, float *xs,
                           int32_t *xsum, int IN, int S, void *stream);

/* ---- a4-a8: decode GEMV family (S = 1..16 rows; any S >= 1 is accepted) --------------------------
 * Replaces launch_gemv_w4a8 / _mlp<U> / _mlp_auto / _g4 (kernels/gemv_w4a8.cuh:93,102,155,316; their
 * unused xsum argument is dropped), launch_gemv_w4a8_sb / _sb_g4 (:168,:337) and
 * launch_gemm_batch_w4a8 (kernels/gemm_batch.cuh:228).
 * Y[s,o] = sum_b xs[s,b]*sw[o,b] * sum_{k in b} xq[s,k]*(Wq[o,k]-8).  Weights are streamed once for
 * all S rows.  Integer group dots are exact; every row's fp32 result is independent of S and of the
 * row's position, and bitwise reproducible. */
int w4a8_gemv(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
              int IN, int OUT, int S, int scale_dtype, void *stream);

/* Several matrices against the SAME activation rows in one call (gate + up, q + k + v: the pairs that share one
 * quantized input in the graphs, models/qwen35_decode.cu:215 "n2 quantized once, shared by gate/up", G4_QUANT_SHARE in
 * models/gemma4_decode.cu:110-112).  Y[i][S, OUT[i]] = w4a8_gemv(xq, xs, Wq[i], sw[i]) for i < count <= 4, bit for bit.
 * A single row whose matrices all qualify for the bulk-copy streaming kernel goes out as ONE kernel launch with the
 * SMs divided between the matrices in proportion to their rows; anything else is the same as `count` calls. */
int w4a8_gemv_multi(const int8_t *xq, const float *xs, int count, const uint8_t *const *Wq,
                    const void *const *sw, float *const *Y, const int *OUT, int IN, int S, int scale_dtype,
                    void *stream);

/* ---- a9-a12: prefill / verify GEMM family ---------------------------------------------------------
 * Replaces launch_gemm_mmq_w4a8 / _kt<KT> / _auto, launch_gemm_mmq_tmpl<...>
 * (kernels/gemm_mmq.cuh:222-233, gemm_mmq_tmpl.cuh:100-119), launch_gemm_mmq_raster_w4a8
 * (kernels/gemm_mmq_raster.cuh:115-130), launch_gemm_mma_w4a8 / _bm<BM> (kernels/gemm_mma.cuh:119-132)
 * and launch_gemm_mmq_ms (kernels/gemm_mmq_ms.cuh).  Note the (M,N,K) argument order of this family.
 * Y[M,N] fp32 row-major.  Integer group dots come from tcgen05 kind::i8 MMAs and are exact; the fp32
 * epilogue evaluates t = (float)D*xs[m,b]; acc = fma(t, sw[n,b], acc) for b ascending, the order of
 * kernels/gemm_mmq.cuh:104-105, so results match the reference MMQ kernels bit for bit.
 * Needs X and Wq 16-byte aligned (TMA); M, N arbitrary. */
int w4a8_gemm(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
              int M, int N, int K, int scale_dtype, void *stream);

/* ---- a13: split-K GEMM for skinny M -----------------------------------------------------------------
 * Replaces launch_gemm_bm16_splitk (kernels/gemm_mmq.cuh:205-219), whose workspace is a grow-only
 * static cudaMalloc inside the launcher (:206,:215; not capture-safe).  Here the caller owns it.
 * K is cut into `splitk` contiguous ranges of ceil(ceil(K/64)/splitk) 64-wide K-tiles; each range is
 * summed in MMQ order into workspace[split][M][N]; a second kernel adds the partials in ascending
 * split order.  splitk <= 0 picks the reference's heuristic (about 96 CTAs, clamp 1..8). */
size_t w4a8_gemm_splitk_workspace_bytes(int M, int N, int K, int splitk);
int w4a8_gemm_splitk(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                     int M, int N, int K, int scale_dtype, int splitk,
                     void *workspace, size_t workspace_bytes, void *stream);

/* ---- split-K GEMM for callers that cannot allocate device memory ------------------------------------
 * No counterpart in the reference (its split-K launcher allocates its own workspace with cudaMalloc,
 * kernels/gemm_mmq.cuh:206,215).
 * Same product and same bits as w4a8_gemm_splitk, but the partial sums live in a fixed buffer that is part
 * of the library image (W4A8_SPLITK_STATIC_BYTES of device memory, held by every GPU that loads the library
 * until the process exits), so the call needs no workspace argument and performs no cudaMalloc / cudaFree
 * or any other allocation.  It is meant for callers that have no way to obtain device scratch at the point
 * of the call: a serving loop that must not touch the device allocator once it is running (an allocation
 * can synchronise the device or fail under memory pressure in the middle of a request), or a host plugin
 * that another runtime handed only its input and output buffers and that owns no allocator of its own.
 *  - Limit: nsplit * M * N * 4 bytes must fit in W4A8_SPLITK_STATIC_BYTES (nsplit as chosen by `splitk`,
 *    see w4a8_gemm_splitk); larger problems are rejected with W4A8_ERR_UNSUPPORTED and a message that names
 *    both sizes.  Use w4a8_gemm_splitk with your own workspace for those.
 *  - The first call on each device looks up the buffer's device address (one host-side query, result
 *    cached per device).  Make that first call outside any stream capture.
 *  - All calls share the one buffer and it keeps whatever the previous call left.  Nothing in it has to be
 *    cleared: the first kernel of a call rewrites every partial sum that the second kernel of the same
 *    call reads.  Because the buffer is shared, two calls whose kernels may overlap on the GPU (different
 *    streams, or concurrent host threads) race on it; issue calls on one stream, or order them yourself. */
#define W4A8_SPLITK_STATIC_BYTES (16u * 1024u * 1024u)
int w4a8_gemm_splitk_static(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, float *Y,
                            int M, int N, int K, int scale_dtype, int splitk, void *stream);

/* ---- exact integer group dots (debug / parity) ------------------------------------------------------
 * D[m,n,b] = sum_{k in b} xq[m,k]*(Wq[n,k]-8) as int32, D laid out [M][N][K/32].  `path` selects the
 * producer: 0 = the GEMV kernels' dp4a path, 1 = the int8 GEMM kernel's tcgen05 kind::i8 path (accumulators
 * read back from tensor memory), 2 = the fp16-operand GEMM kernel's kind::f16 path (fp32 accumulators, exact,
 * converted back to int32).  Checks the bit-exactness the fp32 entry points rest on
 * (tests/test_mma_b0.cu:46-49). */
int w4a8_group_dots(const int8_t *xq, const uint8_t *Wq, int32_t *D, int M, int N, int K, int path,
                    void *stream);

/* ---- mm(): quantize + matmul dispatch ---------------------------------------------------------------
 * Replaces the static mm()/MMs()/mmb() dispatchers of the model graphs (models/qwen35_decode.cu:51-62,
 * models/qwen35_batch.cu:120-139, models/gemma4_decode.cu:113-129): quantize X[S,K] into the caller's
 * scratch (xq, xs, xsum as for w4a8_quantize_x_q8) unless skip_quantize != 0 (the G4_QUANT_SHARE case,
 * models/gemma4_decode.cu:115), then S <= 16 -> w4a8_gemv, else -> w4a8_gemm. */
int w4a8_linear(const float *X, int8_t *xq, float *xs, int32_t *xsum, const uint8_t *Wq, const void *sw,
                float *Y, int S, int N, int K, int scale_dtype, int skip_quantize, void *stream);

/* mm() for a caller whose activations and results live in HOST memory (the daemon side of the reference's pipe
 * protocol, runtime/serving_online.h): copies X_host[S,K] to X_dev, runs w4a8_linear into Y_dev, copies Y_dev[S,N]
 * to Y_host and synchronises the stream, so Y_host is complete on return.  All device buffers are the caller's
 * (same scratch as w4a8_linear plus X_dev and Y_dev); pinned host memory makes the copies asynchronous, and a
 * small pinned X (up to 1 MiB) is read by the quantizer directly over the bus instead of being copied first
 * (X_dev is then unused). */
int w4a8_linear_host(const float *X_host, float *Y_host, float *X_dev, int8_t *xq, float *xs, int32_t *xsum,
                     float *Y_dev, const uint8_t *Wq, const void *sw, int S, int N, int K, int scale_dtype,
                     void *stream);

/* ---- grouped experts (W4A8 semantics per expert) ----------------------------------------------------
 * The reference's expert kernels take fp32 activations (kernels/moe_fused.cuh:14-33); this keeps their
 * weight indexing — expert e starts e*(N*K/2) bytes into Wq and e*(N*K/32) scales into sw
 * (kernels/moe_fused.cuh:21-24), slot = token*topk + k, expert id idx[slot] read on the device (idx may be
 * written by an earlier kernel of the same stream: the kernels wait for that dependency before their first read of
 * it) — and applies the dense W4A8 product per slot.  Y[nslots,N].  x_per_slot = 0: activations are per token
 * (row slot/topk; gate/up projection); 1: per slot (down projection). */
int w4a8_moe_gemv(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, const int32_t *idx,
                  float *Y, int nslots, int topk, int x_per_slot, int N, int K, int num_experts,
                  int scale_dtype, void *stream);

/* ---- routed-expert MLP block (W4A8) ------------------------------------------------------------------
 * Replaces the four launches of the reference's fused expert path at its call site (models/moe_block.cuh:45-52:
 * launch_moe_fused_gu, _swiglu, _down, _reduce; kernels/moe_fused.cuh:14-76) — same tensors, same slot order, same
 * fixed-order combine — with the expert products in W4A8 arithmetic (the reference's are W4A32):
 *   xq, xs      = quantize_x_q8(n2)                                   per token, H elements
 *   gu[slot]    = W4A8 product of token slot/topk with experts_gate_up[idx[slot]]      [2*MI] (gate rows, then up rows)
 *   hid[slot]   = act(gu[slot][0:MI]) * gu[slot][MI:2*MI], quantized per 32-element block
 *   so[slot]    = W4A8 product of hid[slot] with experts_down[idx[slot]]               [H]
 *   out[b]      = sum over k ascending, from 0, of dw[b*topk+k] * so[b*topk+k]         (each product rounded once)
 * gu_wq / gu_sc: flat [E][2*MI][H/2] bytes and [E][2*MI][H/32] scales; dn_wq / dn_sc: [E][H][MI/2], [E][H][MI/32]
 * (runtime/weights_qwen.cu:62-63).  idx (global expert ids) and dw (router weights) are device arrays of S*topk
 * entries written by earlier work of the stream; every id must name an existing expert.
 * Up to 128 slots run as one grouped GEMV launch per projection (with H <= 2048 and MI = 768 those two launches also
 * produce their own activation rows — quantize_x of the token, activation + quantize_x of the slot's gate|up row — and
 * store them to the same xq / xs / xq_h / xs_h stages; on an expert shard the stage rows of tokens and slots whose
 * experts all live on other ranks stay unwritten); above that the slots are sorted by expert on the
 * device and both projections run as grouped tensor-core GEMMs whose work units are (expert, up to 64 of its
 * rows) x 128 outputs (w4a8_config("moe_kernel", 1 | 2) forces one).  Nothing is allocated: the intermediates live
 * in the caller's workspace at the offsets w4a8_moe_layout_for reports (256-byte aligned device memory of
 * layout.bytes bytes).  H and MI multiples of 32, at most 1024 experts. */
typedef struct {
    size_t perm, pos, offsets, items, num_items;  /* sort: sorted row -> slot; slot -> sorted row (-1: another rank's);
                                                     first sorted row per local expert [experts+1]; int4 item list; its length */
    size_t xq, xs;                                /* quantized tokens [S][H] int8, [S][H/32] fp32 */
    size_t xq_g, xs_g;                            /* the same, gathered per sorted row [S*topk][H] (GEMM path) */
    size_t gu;                                    /* [S*topk][2*MI] fp32; rows in sorted order (GEMM path) or slot order (GEMV path) */
    size_t xq_h, xs_h;                            /* quantized hidden [S*topk][MI] int8, [S*topk][MI/32] fp32, same row order */
    size_t sout;                                  /* down outputs [S*topk][H] fp32, same row order, router weight not applied */
    size_t bytes;
} w4a8_moe_layout;
int w4a8_moe_layout_for(int S, int topk, int H, int MI, int experts, w4a8_moe_layout *out);
int w4a8_moe_block(const float *n2, const uint8_t *gu_wq, const void *gu_sc, const uint8_t *dn_wq, const void *dn_sc,
                   const int32_t *idx, const float *dw, float *out, int S, int topk, int H, int MI, int num_experts,
                   int scale_dtype, int act, void *workspace, size_t workspace_bytes, void *stream);
/* Expert-sharded form (new for multi-GPU; nothing in the reference): this rank holds experts
 * [expert_base, expert_base + experts_local) — gu_wq etc. point at ITS experts — and n2, idx, dw are replicated.
 * The rank computes only the slots routed to its experts, stores their down outputs into row `slot` of a
 * slot-ordered buffer Sout[S*topk][H] at sout_offset in EVERY rank's arena (16-byte peer stores), publishes `epoch`,
 * waits (bounded by timeout_us) for every rank's flag and then combines: every rank ends with the whole out[S][H],
 * bit-identical to w4a8_moe_block with all experts on one GPU.  With few slots (grouped-GEMV path and S*topk*H <= 512 Ki)
 * the rows travel as tagged 8-byte stores into the arenas' slot buffers instead and the combine polls for them — no
 * fence, no flag, the Sout buffer at sout_offset is not touched (same rule as w4a8_gemv_allgather_sync: every
 * all-gather step on the arena complete on the stream before the next one is issued).  Arena rules as for w4a8_gemv_allgather (alternate
 * sout_offset between consecutive steps); workspace from w4a8_moe_layout_for(S, topk, H, MI, experts_local).
 * phase 0: the whole block.  phase 1: everything up to and including the publish (no wait, no combine) and
 * phase 2: wait + combine only — for a caller that puts other work between the two, and for several ranks driven
 * one after the other on one GPU, where a kernel must not wait for a rank that has not been launched yet. */
int w4a8_moe_block_shard(const float *n2, const uint8_t *gu_wq, const void *gu_sc, const uint8_t *dn_wq, const void *dn_sc,
                         const int32_t *idx, const float *dw, float *out, int S, int topk, int H, int MI, int expert_base,
                         int experts_local, int scale_dtype, int act, void *workspace, size_t workspace_bytes,
                         struct w4a8_arena *a, size_t sout_offset, uint32_t epoch, int timeout_us, int phase, void *stream);

/* ---- a15: N-sharded weight upload --------------------------------------------------------------------
 * Replaces QMat + load_dev()/mat() (runtime/weights_qwen.h:8, runtime/weights_qwen.cu:12-36,
 * runtime/weights_gemma4.cu:12-41): `<name>_q4.bin` holds N*K/2 bytes, `<name>_scale.bin` holds
 * N*K/32 scales of 4 (scale_dtype 0) or 2 (scale_dtype 1) bytes.  Rank r of `world` keeps rows
 * [row0, row0+rows) — a contiguous byte range of each file, because rows are the outer dimension —
 * on the current device.  world = 1 reproduces the reference's whole-file upload. */
typedef struct w4a8_qmat {
    uint8_t *wq;     /* device, rows*K/2 bytes */
    void *sc;        /* device, rows*K/32 scales */
    int64_t row0;    /* first row held */
    int64_t rows;    /* number of rows held */
    int64_t N, K;    /* full shape */
    int scale_dtype; /* 0 fp32, 1 fp16 */
} w4a8_qmat;

/* Row range of `rank`: floor(N/world) rows each, the remainder spread one row each over the LAST
 * ranks; ranges are contiguous and ordered by rank. */
int w4a8_shard_rows(int64_t N, int rank, int world, int64_t *row0, int64_t *rows);
int w4a8_load_qmat_shard(const char *q4_path, const char *scale_path, int64_t N, int64_t K,
                         int scale_dtype, int rank, int world, w4a8_qmat *out);
/* Same, from host memory holding the full [N] tensors (for callers that already read the files). */
int w4a8_upload_qmat_shard(const uint8_t *host_wq, const void *host_sc, int64_t N, int64_t K,
                           int scale_dtype, int rank, int world, w4a8_qmat *out);
int w4a8_free_qmat(w4a8_qmat *m);

/* ---- N-sharded GEMV with the all-gather fused into the epilogue ------------------------------------------
 * New for multi-GPU; the reference is single-GPU and has nothing to replace here.  One process per GPU.
 * Every rank owns an ARENA: device memory that all ranks of the box map (CUDA IPC, or any other peer mapping the
 * caller has), holding the gathered outputs, a small tail of flags and two internal slot buffers (8 MiB together,
 * allocated behind the `bytes` the caller asks for).  w4a8_gemv_allgather runs the ordinary GEMV on the rank's row
 * shard into the rank's own arena at the final address of Y[M, ldY]; the slice reaches the same place in every
 * other rank's arena through ordinary peer stores over NVLink (no collective, no TMA: from the computing threads
 * for a small slice, from a copy kernel many CTAs wide with row-contiguous 16-byte stores for a large one), and
 * the last CTA publishes `epoch` in a flag on every rank behind one system-scope fence.  w4a8_allgather_wait
 * enqueues a kernel that waits until all ranks' flags in the local arena have reached `epoch`; work enqueued after
 * it on the same stream sees the complete Y.
 * The wait is bounded: after timeout_us it records a device error (w4a8_device_status returns W4A8_ERR_DEVICE)
 * and returns, leaving the context usable.
 * Rules: epochs of successive steps must increase; a rank may start step e+1 only after step e is complete on its
 * stream (w4a8_allgather_wait, or a `_sync` call, in stream order), and Y buffers of consecutive steps must
 * alternate between two offsets, because a fast rank's step e+1 stores may land while a slow rank still reads
 * step e.  Every rank passes the same S, IN, ldY and scale_dtype and equally aligned pointers.  At most 8 ranks.
 * Environment W4A8_ALLGATHER = push | flags | scatter forces one exchange (measurement only). */
typedef struct w4a8_arena w4a8_arena;
int w4a8_arena_create(size_t bytes, int rank, int world, w4a8_arena **out);   /* cudaMalloc'd, zeroed */
void *w4a8_arena_base(w4a8_arena *a);                                          /* local device pointer */
/* bases[r] = arena base of rank r as mapped into THIS process (bases[rank] is ignored and taken as local). */
int w4a8_arena_connect(w4a8_arena *a, void *const *bases);
int w4a8_arena_destroy(w4a8_arena *a);
/* CUDA IPC helpers for the mapping: export the local arena's 64-byte handle, open / close a peer's. */
int w4a8_ipc_export(void *dev_ptr, unsigned char handle[64]);
int w4a8_ipc_open(const unsigned char handle[64], void **dev_ptr);
int w4a8_ipc_close(void *dev_ptr);
/* Y lives at byte offset y_offset in every arena, row pitch ldY floats; this rank writes columns
 * [row0, row0+rows).  Other arguments as w4a8_gemv with OUT = rows. */
int w4a8_gemv_allgather(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a,
                        size_t y_offset, int IN, int rows, int row0, int ldY, int S, int scale_dtype,
                        uint32_t epoch, void *stream);
/* The same for the prefill / verify GEMM (M rows of activations, w4a8_gemm semantics on the rank's `rows` weight rows):
 * the tiles go to columns [row0, row0+rows) of Y[M, ldY] in the rank's own arena, a copy kernel sends the finished
 * slice to the same place in every other rank's arena with row-contiguous 16-byte peer stores, then the epoch is
 * published (environment W4A8_GEMM_ALLGATHER=stores: the GEMM's epilogue stores into every arena itself instead);
 * no split-K.  X and Wq 16-byte aligned as for w4a8_gemm. */
int w4a8_gemm_allgather(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a,
                        size_t y_offset, int M, int rows, int row0, int ldY, int K, int scale_dtype,
                        uint32_t epoch, void *stream);
int w4a8_allgather_wait(w4a8_arena *a, uint32_t epoch, int timeout_us, void *stream);
/* The same two products with the wait folded into their last kernel: when the call's last kernel completes,
 * Y[M, ldY] is complete in this rank's arena and no separate wait kernel sits on the critical path of a decode step.
 * The GEMV with one launch and M*ldY <= 512 Ki outputs uses tagged slots instead of flags: every output also goes,
 * as one 8-byte store {value, tag of the epoch}, into a slot buffer of every other arena, and every CTA, once its
 * rows are done, polls its share of the slots the other ranks fill here and writes them into the local Y — no fence,
 * no flag (such a step does not publish its epoch: do not call w4a8_allgather_wait for it).  Otherwise the CTA that
 * publishes the epoch also waits for every rank's flag.  Either wait gives up after timeout_us (W4A8_ERR_DEVICE
 * through w4a8_device_status).  Every rank of the group must make the matching call: a rank whose peers never
 * arrive only returns after the time-out.  Not for several ranks driven one after the other on one GPU (use
 * w4a8_gemv_allgather + w4a8_allgather_wait there). */
int w4a8_gemv_allgather_sync(const int8_t *xq, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a,
                             size_t y_offset, int IN, int rows, int row0, int ldY, int S, int scale_dtype,
                             uint32_t epoch, int timeout_us, void *stream);
int w4a8_gemm_allgather_sync(const int8_t *X, const float *xs, const uint8_t *Wq, const void *sw, w4a8_arena *a,
                             size_t y_offset, int M, int rows, int row0, int ldY, int K, int scale_dtype,
                             uint32_t epoch, int timeout_us, void *stream);
/* The epoch a kernel publishes / waits for is `epoch` plus a per-arena base kept in device memory (initially 0).
 * This enqueues base += delta.  A CUDA graph that captured steps with epochs 1..n ends with
 * w4a8_arena_advance_epoch(a, n, stream), so that every replay (on all ranks alike) uses fresh epochs. */
int w4a8_arena_advance_epoch(w4a8_arena *a, uint32_t delta, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* W4A8_B200_H */
