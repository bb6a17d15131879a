// Fused GEMV + all-gather for N-sharded weights (no counterpart in the reference, which is single-GPU).
// Every rank holds rows [row0, row0+rows) of Wq / sw and computes Y[:, row0:row0+rows].  Instead of a collective
// after the kernel, the GEMV epilogue stores each output straight into EVERY rank's Y at its final address
// (plain st.global through peer-mapped pointers over NVLink: 4 bytes x world per output, 8.7 KB per peer at M=1),
// and the last CTA to finish publishes a per-rank flag on every peer.  A consumer waits (bounded) until all `world`
// flags of its own arena have reached the step's epoch.  No TMA, no multicast: peer memory is only ever the target
// of ordinary stores and the flags are ordinary release stores / acquire loads.
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

struct OutArgs {                    // passed by value to the GEMV kernels; peers == nullptr: ordinary Y[m*OUT + r]
    const PeerDesc *peers = nullptr;
    size_t y_off = 0;               // byte offset of Y[M, ld] inside every arena
    long ld = 0, col0 = 0;          // row pitch of the gathered Y (= total N) and this rank's first column (= row0)
    unsigned int epoch = 0;         // value published in the flags when this launch's stores are complete
    int publish = 0;                // 1: the last CTA of this launch publishes; 0: a later launch of the same call does
    int local_only = 0;             // 1 (GEMM): store only into this rank's own arena; allgather_scatter_kernel sends the slice on
};

// PEER is a template parameter of the GEMV kernels: the single-GPU instantiation carries none of this code.
template <bool PEER>
__device__ __forceinline__ void store_out(float *Y, const OutArgs &oa, int OUT, int m, int r, float v) {
    if (!PEER) { Y[(size_t)m * OUT + r] = v; return; }
    const PeerDesc *p = oa.peers;
    const int world = p->world;
    for (int k = 0; k < world; k++)
        reinterpret_cast<float *>(p->base[k] + oa.y_off)[(size_t)m * oa.ld + oa.col0 + r] = v;
}

// Called by every thread of every CTA after its last store; `stored` = this thread wrote outputs (only those
// threads pay for the system-scope fence).
template <bool PEER>
__device__ __forceinline__ void publish_out(const OutArgs &oa, bool stored = true) {
    if (!PEER || !oa.publish) return;
    if (stored) __threadfence_system();            // this thread's peer stores are visible system-wide
    __syncthreads();
    if (threadIdx.x == 0) {
        const PeerDesc *p = oa.peers;
        const unsigned total = gridDim.x * gridDim.y;
        const unsigned prev = atomicAdd(p->counter, 1u);
        if (prev == total - 1) {                   // last CTA: all CTAs' stores are fenced
            *p->counter = 0u;
            __threadfence_system();
            const unsigned int e = *p->epoch_base + oa.epoch;
            for (int k = 0; k < p->world; k++) {
                unsigned int *f = reinterpret_cast<unsigned int *>(p->base[k] + p->flag_off) + p->rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(e) : "memory");
            }
        }
    }
}

// Publishes `epoch` after earlier launches of the same stream (which stored without publishing) have completed.
__global__ void allgather_publish_kernel(const PeerDesc *p, unsigned int epoch) {
    if (threadIdx.x != 0) return;
    __threadfence_system();
    epoch += *p->epoch_base;
    for (int k = 0; k < p->world; k++) {
        unsigned int *f = reinterpret_cast<unsigned int *>(p->base[k] + p->flag_off) + p->rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(epoch) : "memory");
    }
}

// One warp; lane r < world waits until rank r's flag in THIS rank's arena has reached `epoch`.  Bounded: after
// `limit_cycles` SM clocks the lane gives up and records an error (w4a8_device_status) instead of spinning on.
__global__ void allgather_wait_kernel(const PeerDesc *p, unsigned int epoch, long long limit_cycles) {
    const int r = threadIdx.x;
    // Launched for programmatic dependent launch: resident early, and the kernel after it (typically the next GEMV,
    // which may prefetch weights) may become resident too; polling starts only once this rank's own producer kernel
    // has completed, so the only flags still outstanding are the ones other GPUs write.
    pdl_launch_dependents();
    pdl_wait();
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

// Sends this rank's finished slice Y[0..M, col0..col0+cols) of its OWN arena to the same place in every other rank's
// arena and publishes `epoch`.  Consecutive lanes copy consecutive 16-byte pieces of a row, so the NVLink writes are
// whole rows' worth of contiguous bytes (the GEMM's own epilogue can only offer 16-byte pieces of 32 different rows
// per instruction, which reached about 300 GB/s).  Needs col0, cols and ld multiples of 4 for the 16-byte path.
__global__ void __launch_bounds__(256) allgather_scatter_kernel(const PeerDesc *p, size_t y_off, int M, long ld, long col0, int cols,
                                                                unsigned int epoch) {
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
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned prev = atomicAdd(p->counter, 1u);
        if (prev == gridDim.x - 1) {               // last CTA: every CTA's stores are fenced
            *p->counter = 0u;
            __threadfence_system();
            const unsigned int e = *p->epoch_base + epoch;
            for (int k = 0; k < world; k++) {
                unsigned int *f = reinterpret_cast<unsigned int *>(p->base[k] + p->flag_off) + rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f), "r"(e) : "memory");
            }
        }
    }
}

// epoch_base += delta: the last node of a captured graph of `delta` steps, so that the next replay of the same graph
// publishes and waits for fresh epochs.
__global__ void allgather_advance_kernel(const PeerDesc *p, unsigned int delta) {
    if (threadIdx.x == 0) *p->epoch_base += delta;
}

}  // namespace w4a8
