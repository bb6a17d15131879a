// Fused GEMV + all-gather for N-sharded weights (no counterpart in the reference, which is single-GPU).
// Every rank holds rows [row0, row0+rows) of Wq / sw and computes Y[:, row0:row0+rows] into its OWN arena at the final
// address.  The last CTA of the launch to finish (a counter in the arena) then pushes the rank's finished slice to the
// same place in every other rank's arena — consecutive lanes write consecutive 16-byte pieces of a row, so NVLink
// sees whole rows, 8.7 KB per peer at M=1 with 8 ranks —, issues ONE system-scope fence and publishes a per-rank flag
// on every peer.  (Storing every output to every peer from the thread that computed it, each followed by its own
// system fence, cost 14 us per step at 2 ranks and 27 us at 8.)  A slice too large for one CTA to push (more than
// PUSH_MAX_BYTES over all peers) is sent by allgather_scatter_kernel instead, many CTAs wide.  A consumer waits
// (bounded) until all `world` flags of its own arena have reached the step's epoch: either a small kernel of its own
// (w4a8_allgather_wait), or — oa.wait_limit > 0 — the pushing CTA itself before it exits, so that the completion of
// the launch means "Y is complete on this rank" and no extra launch sits on the critical path of a decode step.
// No TMA, no multicast: peer memory is only ever the target of ordinary stores and the flags are ordinary release
// stores / acquire loads.
//
// Arena layout (one per rank, same size everywhere): [ user bytes ... | 256-byte tail: flags[8], counter, epoch base ].
#pragma once
#include "common.cuh"

namespace w4a8 {

constexpr int PEER_MAX = 8;
constexpr size_t PEER_TAIL = 256;

struct PeerDesc {                   // lives in device memory of the owning rank
    unsigned char *base[PEER_MAX];  // arena base of every rank as mapped into this process (base[rank] = local)
    unsigned int *counter;          // local: CTAs of the running kernel that have finished their stores
    unsigned int *epoch_base;       // local: added to every epoch argument (lets a captured graph be replayed)
    size_t flag_off;                // byte offset of flags[] inside every arena
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
};

// PEER is a template parameter of the GEMV kernels: the single-GPU instantiation carries none of this code.
template <bool PEER>
__device__ __forceinline__ void store_out(float *Y, const OutArgs &oa, int OUT, int m, int r, float v) {
    if (!PEER) { Y[(size_t)m * OUT + r] = v; return; }
    const PeerDesc *p = oa.peers;
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
    for (long i = threadIdx.x; i < total; i += blockDim.x) {
        const long m = i / per_row, c = i - m * per_row;
        if (v4) {
            const size_t off = (size_t)m * ld + col0 + 4 * c;
            const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + off));   // written by other CTAs: read at L2
            for (int k = 0; k < world; k++)
                if (k != rank) *reinterpret_cast<float4 *>(reinterpret_cast<float *>(p->base[k] + y_off) + off) = v;
        } else {
            const size_t off = (size_t)m * ld + col0 + c;
            const float v = __ldcg(src + off);
            for (int k = 0; k < world; k++)
                if (k != rank) reinterpret_cast<float *>(p->base[k] + y_off)[off] = v;
        }
    }
}

// Thread 0 of the publishing CTA, after a CTA barrier behind the last peer store: one system-scope fence (cumulative
// over the stores the barrier ordered before it), then this rank's flag in every arena.
__device__ __forceinline__ void publish_flags(const PeerDesc *p, unsigned int epoch) {
    __threadfence_system();
    const unsigned int e = *p->epoch_base + epoch;
    for (int k = 0; k < p->world; k++) {
        unsigned int *f = reinterpret_cast<unsigned int *>(p->base[k] + p->flag_off) + p->rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(e) : "memory");
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
    for (;;) {
        unsigned int v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if ((int)(v - epoch) >= 0) return;
        if (clock64() - t0 > limit_cycles) { dev_set_error(0x200u | (unsigned)r); return; }
    }
}

// Called by every thread of every CTA after its last store; `stored` = this thread wrote outputs.
template <bool PEER>
__device__ __forceinline__ void publish_out(const OutArgs &oa, bool stored = true) {
    if (!PEER || !oa.publish) return;
    const PeerDesc *p = oa.peers;
    // this thread's stores are visible: device-wide when they went to the rank's own arena, system-wide when it wrote to peers
    if (stored) { if (oa.local_only) __threadfence(); else __threadfence_system(); }
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
