// Common part of the drop-in launcher shims: each shim header in this directory carries the name of the
// reference header it replaces (kernels/quantize_x.cuh, gemv_w4a8.cuh, gemm_batch.cuh, gemm_mma.cuh,
// gemm_mmq.cuh, gemm_mmq_tmpl.cuh, gemm_mmq_raster.cuh, qscale.cuh, reduce.cuh) and defines the same
// `static inline void launch_*` functions, forwarding to the C ABI of libw4a8_b200.so.  Put this directory
// ahead of the reference's kernels/ on the include path and link -lw4a8_b200; models/*.cu compile unchanged.
//
// The reference launchers return void and never look at errors; its callers synchronise and exit(1) on any CUDA
// error (models/qwen35_decode.cu:24-25,229).  A failed ABI call is therefore reported the same way: message on
// stderr, exit(1).  Define W4A8_SHIM_NO_EXIT to ignore failures instead.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include "../../include/w4a8_b200.h"

#ifndef QBLK
#define QBLK W4A8_QBLK   // runtime/config.h:9-11
#endif

static inline void w4a8_shim_check(int rc, const char *what) {
    if (rc == W4A8_OK) return;
    fprintf(stderr, "w4a8 %s failed (%d): %s\n", what, rc, w4a8_last_error());
#ifndef W4A8_SHIM_NO_EXIT
    exit(1);
#endif
}
