// Drop-in proof: the reference's OWN unit test tests/test_w4a8.cu, compiled unmodified from where it lies, but with
// this repository's shim launchers standing in for kernels/quantize_x.cuh and kernels/gemv_w4a8.cuh.  The shims are
// included first; defining the reference headers' include guards makes the test's own #include lines no-ops.
// Built by oracle/Makefile into oracle/_ref/ (git-ignored); run by tests/test_gpu_vs_reference.py.
#include "quantize_x.cuh"     // dgx-serving_b200/kernels (via -I)
#include "gemv_w4a8.cuh"
#define DGX_QUANTIZE_X_CUH
#define DGX_GEMV_W4A8_CUH
#include "tests/test_w4a8.cu" // reference tree (via -I)
