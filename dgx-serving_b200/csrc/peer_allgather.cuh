// Fused GEMV / GEMM + all-gather for N-sharded weights (no counterpart in the reference, which is single-GPU).
// Every rank holds rows [row0, row0+rows) of Wq / sw, computes Y[:, row0:row0+rows] and every rank ends up with the
// whole Y[M, N] in its own arena.  Two exchanges, chosen by the host from the size of the slice:
//
//  * tagged slots (decode: one launch, a small Y, the `_sync` entry points).  The thread that computed an output
//    stores it into its own arena's Y and, as ONE 8-byte store {value, tag of the step}, into a slot buffer of every
//    other arena.  8-byte stores are single-copy atomic, so a reader that sees the step's tag has the value: no fence,
//    no flag, no "last CTA".  When a CTA has finished its rows it polls (bounded) its share of the slots other ranks
//    fill in this rank's arena and writes the values into the local Y; when the launch completes, Y is complete here.
//    Two slot buffers alternate with the step's epoch: a rank can only be one step ahead of a peer (it cannot finish
//    step e+1 without that peer's step-e+1 outputs, which the peer sends after it has finished reading step e), so a
//    buffer is never overwritten while someone still reads it — provided every all-gather step issued on the arena is
//    complete on the stream (in-kernel or by w4a8_allgather_wait) before the next tagged step is issued.
//    Fences were what made the flag protocol slow at this size: a system-scope fence behind remote stores waits for
//    their NVLink round trip (2.4 us measured), and so does the device-scope fence of every storing thread.
//
//  * slice + flags (everything else).  Outputs go to the rank's own arena; a small slice is also stored to every other
//    arena by the computing threads themselves (W4A8_ALLGATHER=push: copied by the last CTA instead), a large one is
//    sent afterwards with row-contiguous 16-byte stores (allgather_scatter_kernel, many CTAs); the last CTA issues ONE
//    system-scope fence and publishes a per-rank flag on every peer with relaxed stores.  A consumer waits (bounded) until all `world` flags of its own arena have reached the
//    step's epoch: a small kernel of its own (w4a8_allgather_wait) or — oa.wait_limit > 0 — the publishing CTA itself.
//
// No TMA, no multicast: peer memory is only ever the target of ordinary stores.
//
// Arena layout (one per rank, same size everywhere):
//   [ user bytes ... | 256-byte tail: flags[8], counter, epoch base | slot buffer 0 | slot buffer 1 ].
#pragma once
#include "common.cuh"

namespace w4a8 {

constexpr int PEER_MAX = 8;
constexpr size_t PEER_TAIL = 256;
constexpr size_t LL_BUF_BYTES = 4u << 20;          // one slot buffer: 512 Ki outputs of 8 bytes {fp32 bits, tag}
constexpr size_t LL_MAX_SLOTS = LL_BUF_BYTES / 8;

struct PeerDesc {                   // lives in device memory of the owning rank
    unsigned char *base[PEER_MAX];  // arena base of every rank as mapped into this process (base[rank] = local)
    unsigned int *counter;          // local: CTAs of the running kernel that have finished their stores
    unsigned int *epoch_base;       // local: added to every epoch argument (lets a captured graph be replayed)
    size_t flag_off;                // byte offset of flags[] inside every arena
    size_t ll_off;                  // byte offset of the two slot buffers inside every arena
    int world, rank;
};

constexpr size_t PUSH_MAX_BYTES = 96 * 1024;   // slice bytes x (world - 1) that one CTA may push itself

struct OutArgs {                    // passed by value to the GEMV kernels; peers == nullptr: ordinary Y[m*OUT + r]
    const PeerDesc *peers = nullptr;
    size_t y_off = 0;               // byte offset of Y[M, ld] inside every arena
    long ld = 0, col0 = 0;          // row pitch of the gathered Y (= total N) and this rank's first column (= row0)
    unsigned int epoch = 0;         // value published in the flags when this launch's stores are complete
    int publish = 0;                // 1: the last CTA of this launch sends the slice on (push) and publishes; 0: a later launch does
    int local_only = 1;             // 1: store only into this rank's own arena (the slice is sent on afterwards); 0: every
                                    //    output goes to every arena from the thread that computed it (GEMM, W4A8_GEMM_ALLGATHER=stores)
    int push = 0;                   // 1: the last CTA copies Y[0..M, col0..col0+cols) to every other arena before it publishes
    int M = 0, cols = 0;            // shape of this rank's slice (push)
    long long wait_limit = 0;       // > 0: the last CTA also waits (at most this many SM clocks) for every rank's flag
    int ll = 0;                     // 1: tagged-slot exchange (see the top of this file); wait_limit bounds every poll
};

// Tag of a step in the slot buffers: never 0, the value the arena is created with, for any epoch below 2^32 - 1.
__device__ __forceinline__ unsigned int ll_tag(unsigned int e) { return ~e; }

// PEER is a template parameter of the GEMV kernels: the single-GPU instantiation carries none of this code.
template <bool PEER>
__device__ __forceinline__ void store_out(float *Y, const OutArgs &oa, int OUT, int m, int r, float v) {
    if (!PEER) { Y[(size_t)m * OUT + r] = v; return; }
    const PeerDesc *p = oa.peers;
    if (oa.ll) {
        const size_t idx = (size_t)m * oa.ld + oa.col0 + r;
        const int world = p->world, rank = p->rank;
        reinterpret_cast<float *>(p->base[rank] + oa.y_off)[idx] = v;
        const unsigned int e = *p->epoch_base + oa.epoch;
        const unsigned long long pk = ((unsigned long long)ll_tag(e) << 32) | (unsigned long long)__float_as_uint(v);
        const size_t off = p->ll_off + (size_t)(e & 1u) * LL_BUF_BYTES + idx * 8;
        for (int k = 0; k < world; k++)
            if (k != rank) asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p->base[k] + off), "l"(pk) : "memory");
        return;
    }
    if (oa.local_only) {
        reinterpret_cast<float *>(p->base[p->rank] + oa.y_off)[(size_t)m * oa.ld + oa.col0 + r] = v;
        return;
    }
    const int world = p->world;
    for (int k = 0; k < world; k++)
        reinterpret_cast<float *>(p->base[k] + oa.y_off)[(size_t)m * oa.ld + oa.col0 + r] = v;
}

// All threads of one CTA: copy this rank's slice Y[0..M, col0..col0+cols) of its own arena to every other arena.
__device__ __forceinline__ void push_slice(const PeerDesc *p, size_t y_off, int M, long ld, long col0, int cols) {
    const int world = p->world, rank = p->rank;
    const float *src = reinterpret_cast<const float *>(p->base[rank] + y_off);
    const bool v4 = ((ld | col0 | cols) & 3) == 0;
    const long per_row = v4 ? cols / 4 : cols, total = (long)M * per_row;
    if (v4) {
        // batches of UB loads in flight per thread: a load is an L2 round trip, a dozen of them one after the other
        // would cost more than the whole exchange
        constexpr int UB = 8;
        for (long i0 = threadIdx.x; i0 < total; i0 += (long)blockDim.x * UB) {
            float4 v[UB];
            size_t off[UB];
#pragma unroll
            for (int u = 0; u < UB; u++) {
                const long i = i0 + (long)u * blockDim.x;
                if (i < total) {
                    const long m = i / per_row, c = i - m * per_row;
                    off[u] = (size_t)m * ld + col0 + 4 * c;
                    v[u] = __ldcg(reinterpret_cast<const float4 *>(src + off[u]));   // written by other CTAs: read at L2
                }
            }
#pragma unroll
            for (int u = 0; u < UB; u++) {
                if (i0 + (long)u * blockDim.x < total) {
                    for (int k = 0; k < world; k++)
                        if (k != rank) *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p->base[k] + y_off) + off[u]) = v[u];
                }
            }
        }
    } else {
        for (long i = threadIdx.x; i < total; i += blockDim.x) {
            const long m = i / per_row, c = i - m * per_row;
            const size_t off = (size_t)m * ld + col0 + c;
            const float v = __ldcg(src + off);
            for (int k = 0; k < world; k++)
                if (k != rank) reinterpret_cast<float *>(p->base[k] + y_off)[off] = v;
        }
    }
}

// Thread 0 of the publishing CTA, after a CTA barrier behind the last peer store: ONE system-scope fence (cumulative
// over the stores the barrier ordered before it), then this rank's flag in every arena with relaxed stores.  A
// release store per flag would each be a system-scope release of its own, waiting for the acknowledgement of the flag
// store before it: world + 1 fences one after the other, 10 us of a decode step at 2 ranks and 27 us at 8.
__device__ __forceinline__ void publish_flags(const PeerDesc *p, unsigned int epoch) {
    const unsigned int e = *p->epoch_base + epoch;
    __threadfence_system();
    for (int k = 0; k < p->world; k++) {
        unsigned int *f = reinterpret_cast<unsigned int *>(p->base[k] + p->flag_off) + p->rank;
        asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(f), "r"(e) : "memory");
    }
}

// Lane r < world of one warp: wait until rank r's flag in THIS rank's arena has reached `epoch`.  Bounded: after
// `limit_cycles` SM clocks the lane gives up and records an error (w4a8_device_status) instead of spinning on.
__device__ __forceinline__ void wait_flags(const PeerDesc *p, unsigned int epoch, long long limit_cycles) {
    const int r = threadIdx.x & 31;
    if (r >= p->world) return;
    const unsigned int *f = reinterpret_cast<const unsigned int *>(p->base[p->rank] + p->flag_off) + r;
    epoch += *p->epoch_base;
    const long long t0 = clock64();
    for (;;) {                                       // relaxed polls, one acquire fence once the flag is there
        unsigned int v;
        asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if ((int)(v - epoch) >= 0) break;
        if (clock64() - t0 > limit_cycles) { dev_set_error(0x200u | (unsigned)r); return; }
    }
    asm volatile("fence.acq_rel.sys;" ::: "memory");
}

// Tagged-slot exchange, receiving side; every thread of every CTA after its last store.  The M x (ld - cols) outputs
// other ranks compute are dealt out over all threads of the launch; a thread polls its slot in this rank's arena until
// it carries the step's tag (bounded: after wait_limit SM clocks it records error 0x208 and polls the rest of its share
// once each), and writes the value into the local Y.
__device__ __forceinline__ void ll_gather(const OutArgs &oa) {
    const PeerDesc *p = oa.peers;
    const unsigned int e = *p->epoch_base + oa.epoch, tag = ll_tag(e);
    unsigned char *mine = p->base[p->rank];
    const unsigned long long *slots = reinterpret_cast<const unsigned long long *>(mine + p->ll_off + (size_t)(e & 1u) * LL_BUF_BYTES);
    float *Y = reinterpret_cast<float *>(mine + oa.y_off);
    const long per_row = oa.ld - oa.cols, total = (long)oa.M * per_row;
    const long nthr = (long)blockDim.x * blockDim.y * blockDim.z;
    const long tid = threadIdx.x + (long)blockDim.x * (threadIdx.y + (long)blockDim.y * threadIdx.z);
    const long cta = blockIdx.x + (long)gridDim.x * (blockIdx.y + (long)gridDim.y * blockIdx.z);
    const long step = nthr * gridDim.x * gridDim.y * gridDim.z;
    bool gave_up = false;
    for (long i = cta * nthr + tid; i < total; i += step) {
        const long m = i / per_row;
        long c = i - m * per_row;
        if (c >= oa.col0) c += oa.cols;
        const size_t idx = (size_t)m * oa.ld + c;
        const long long t0 = clock64();
        for (;;) {
            unsigned long long v;
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(slots + idx) : "memory");
            if ((unsigned int)(v >> 32) == tag) { Y[idx] = __uint_as_float((unsigned int)v); break; }
            if (gave_up) break;
            if (clock64() - t0 > oa.wait_limit) { dev_set_error(0x208u); gave_up = true; break; }
        }
    }
}

// Called by every thread of every CTA after its last store; `stored` = this thread wrote outputs.
template <bool PEER>
__device__ __forceinline__ void publish_out(const OutArgs &oa, bool stored = true) {
    if (!PEER) return;
    if (oa.ll) { ll_gather(oa); return; }
    if (!oa.publish) return;
    const PeerDesc *p = oa.peers;
    // This thread's stores (to the rank's own arena, or to every arena) are ordered before its CTA's arrival at the
    // counter by a DEVICE-scope fence; the last CTA observes every arrival and then issues one SYSTEM-scope fence, which
    // is cumulative over everything that happened before it, the other CTAs' peer stores included.  (A system-scope
    // fence in every storing thread stalls each of them for a couple of microseconds for nothing.)
    if (stored) __threadfence();
    __syncthreads();
    __shared__ unsigned int s_last;
    if (threadIdx.x == 0) {
        const unsigned total = gridDim.x * gridDim.y;
        s_last = (atomicAdd(p->counter, 1u) == total - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    // last CTA: every CTA's stores are fenced and its arrival at the counter has been observed
    __threadfence();
    if (oa.push) push_slice(p, oa.y_off, oa.M, oa.ld, oa.col0, oa.cols);
    __syncthreads();
    if (threadIdx.x == 0) {
        *p->counter = 0u;
        publish_flags(p, oa.epoch);
    }
    if (oa.wait_limit > 0 && threadIdx.x < 32) wait_flags(p, oa.epoch, oa.wait_limit);
}

// A rank without rows of its own in a tagged-slot step: it only receives.
__global__ void __launch_bounds__(256) allgather_ll_gather_kernel(OutArgs oa) {
    pdl_launch_dependents();
    pdl_wait();                                    // Y of the step before may still be read by the kernel before this one
    ll_gather(oa);
}

// Publishes `epoch` after earlier launches of the same stream (which stored without publishing) have completed;
// wait_limit > 0: also waits for every rank's flag.
__global__ void allgather_publish_kernel(const PeerDesc *p, unsigned int epoch, long long wait_limit) {
    if (threadIdx.x == 0) publish_flags(p, epoch);
    if (wait_limit > 0) wait_flags(p, epoch, wait_limit);
}

// One warp; lane r < world waits until rank r's flag in THIS rank's arena has reached `epoch` (bounded, see wait_flags).
__global__ void allgather_wait_kernel(const PeerDesc *p, unsigned int epoch, long long limit_cycles) {
    // Launched for programmatic dependent launch: resident early, and the kernel after it (typically the next GEMV,
    // which may prefetch weights) may become resident too; polling starts only once this rank's own producer kernel
    // has completed, so the only flags still outstanding are the ones other GPUs write.
    pdl_launch_dependents();
    pdl_wait();
    wait_flags(p, epoch, limit_cycles);
}

// Sends this rank's finished slice Y[0..M, col0..col0+cols) of its OWN arena to the same place in every other rank's
// arena and publishes `epoch`; many CTAs wide, for slices too large for one CTA.  Consecutive lanes copy consecutive
// 16-byte pieces of a row, so the NVLink writes are whole rows' worth of contiguous bytes (the GEMM's own epilogue can
// only offer 16-byte pieces of 32 different rows per instruction, which reached about 300 GB/s).  Needs col0, cols and
// ld multiples of 4 for the 16-byte path.  wait_limit > 0: the last CTA also waits for every rank's flag.
__global__ void __launch_bounds__(256) allgather_scatter_kernel(const PeerDesc *p, size_t y_off, int M, long ld, long col0, int cols,
                                                                unsigned int epoch, long long wait_limit) {
    pdl_launch_dependents();
    pdl_wait();                                    // the slice comes from the kernel before this one
    const int world = p->world, rank = p->rank;
    const float *src = reinterpret_cast<const float *>(p->base[rank] + y_off);
    const bool v4 = ((ld | col0 | cols) & 3) == 0;
    const long per_row = v4 ? cols / 4 : cols, total = (long)M * per_row;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long m = i / per_row, c = i - m * per_row;
        if (v4) {
            const size_t off = (size_t)m * ld + col0 + 4 * c;
            const float4 v = *reinterpret_cast<const float4 *>(src + off);
            for (int k = 0; k < world; k++)
                if (k != rank) *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p->base[k] + y_off) + off) = v;
        } else {
            const size_t off = (size_t)m * ld + col0 + c;
            const float v = src[off];
            for (int k = 0; k < world; k++)
                if (k != rank) reinterpret_cast<float *>(p->base[k] + y_off)[off] = v;
        }
    }
    __syncthreads();
    __shared__ unsigned int s_last;
    if (threadIdx.x == 0) {
        __threadfence_system();                    // cumulative over this CTA's peer stores (ordered before it by the barrier)
        s_last = (atomicAdd(p->counter, 1u) == gridDim.x - 1) ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    if (threadIdx.x == 0) {                        // last CTA: every CTA's stores are fenced
        *p->counter = 0u;
        publish_flags(p, epoch);
    }
    if (wait_limit > 0 && threadIdx.x < 32) wait_flags(p, epoch, wait_limit);
}

// epoch_base += delta: the last node of a captured graph of `delta` steps, so that the next replay of the same graph
// publishes and waits for fresh epochs.
__global__ void allgather_advance_kernel(const PeerDesc *p, unsigned int delta) {
    if (threadIdx.x == 0) *p->epoch_base += delta;
}

}  // namespace w4a8
