// Drop-in for the reference's kernels/qscale.cuh (:5-6): weight scale read as float, for tools that use it directly.
#pragma once
#include <cuda_fp16.h>
__device__ __forceinline__ float sval(float x) { return x; }
__device__ __forceinline__ float sval(__half x) { return __half2float(x); }
