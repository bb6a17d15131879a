// Drop-in for the part of the reference's kernels/reduce.cuh (:6-9) that tools on the W4A8 path use directly.
#pragma once
__inline__ __device__ float warp_reduce_sum(float v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}
