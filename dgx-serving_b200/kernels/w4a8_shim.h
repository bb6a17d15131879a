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
#include <cstring>
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

// A knob of the reference as its registry resolves it (runtime/knobs.h:9-12, knob_raw :297-303): the environment
// variable, else the last line "NAME=VALUE" of the recipe file named by DGX_KNOBS_FILE ('#' starts a comment, blanks
// around name and value are dropped), else nullptr and the caller applies its default.  Range checks and the
// registry's typo warnings stay with the reference's own runtime/knobs.h; a value below the knob's range is treated
// as unset by the callers here.  Read once per call site (the callers keep the result in a function-scope static,
// as the reference does).
static inline const char *w4a8_shim_knob(const char *name) {
    if (const char *v = getenv(name)) return v;
    const char *path = getenv("DGX_KNOBS_FILE");
    if (!path) return nullptr;
    FILE *f = fopen(path, "r");
    if (!f) { fprintf(stderr, "knobs: cannot read DGX_KNOBS_FILE=%s\n", path); exit(2); }   // runtime/knobs.h:247
    static thread_local char val[256];
    const char *found = nullptr;
    const size_t nl = strlen(name);
    char line[1024];
    while (fgets(line, sizeof line, f)) {
        if (char *h = strchr(line, '#')) *h = 0;
        char *p = line;
        while (*p == ' ' || *p == '\t' || *p == '\r') p++;
        if (strncmp(p, name, nl) != 0) continue;
        char *q = p + nl;
        while (*q == ' ' || *q == '\t') q++;
        if (*q != '=') continue;
        q++;
        while (*q == ' ' || *q == '\t') q++;
        size_t n = strlen(q);
        while (n > 0 && (q[n - 1] == ' ' || q[n - 1] == '\t' || q[n - 1] == '\r' || q[n - 1] == '\n')) n--;
        if (n >= sizeof val) n = sizeof val - 1;
        memcpy(val, q, n);
        val[n] = 0;
        found = val;
    }
    fclose(f);
    return found;
}
