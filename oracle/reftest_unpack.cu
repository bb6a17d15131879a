// Checks the two device helpers the drop-in headers provide for the reference's other files (w4a8_pk of
// kernels/gemv_w4a8.cuh:16-21 and mmq_unpack4v of kernels/gemm_mmq.cuh:25-28) over every 16-bit input against the
// definition "byte i = (4-bit code i) - 8 as a signed byte, low nibble first", evaluated on the host.
// Built by oracle/Makefile into oracle/_ref/; run by tests/test_gpu_vs_reference.py.
#include <cstdio>
#include <vector>
#include "gemv_w4a8.cuh"   // dgx-serving_b200/kernels (via -I)
#include "gemm_mmq.cuh"

__global__ void unpack_all(int *pk, int *un) {
    const unsigned h = blockIdx.x * blockDim.x + threadIdx.x;     // 0 .. 65535
    pk[h] = w4a8_pk((int)(h & 0xFF), (int)((h >> 8) & 0xFF));
    un[h] = mmq_unpack4v(h | 0xABCD0000u);                          // the upper half must be ignored
}

int main() {
    int *pk, *un;
    if (cudaMalloc(&pk, 65536 * 4) != cudaSuccess || cudaMalloc(&un, 65536 * 4) != cudaSuccess) { printf("cudaMalloc failed\n"); return 1; }
    unpack_all<<<256, 256>>>(pk, un);
    std::vector<int> a(65536), b(65536);
    if (cudaMemcpy(a.data(), pk, 65536 * 4, cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy(b.data(), un, 65536 * 4, cudaMemcpyDeviceToHost) != cudaSuccess) { printf("copy failed\n"); return 1; }
    int bad = 0;
    for (unsigned h = 0; h < 65536; h++) {
        unsigned want = 0;
        for (int i = 0; i < 4; i++) want |= (unsigned)((int)((h >> (4 * i)) & 0xF) - 8 & 0xFF) << (8 * i);
        if ((unsigned)a[h] != want || (unsigned)b[h] != want) bad++;
    }
    printf("[reftest_unpack] %s (%d mismatches of 65536)\n", bad ? "FAIL" : "PASS", bad);
    return bad ? 1 : 0;
}
