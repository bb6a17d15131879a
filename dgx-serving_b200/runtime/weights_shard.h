// N-sharded counterpart of the reference's QMat loader (runtime/weights_qwen.h:8, runtime/weights_qwen.cu:12-36,
// runtime/weights_gemma4.cu:12-41).  `mat(name, OUT, IN)` there reads `<dir>/<name>_q4.bin` (OUT*IN/2 bytes) and
// `<dir>/<name>_scale.bin` (OUT*IN/32 scales of 4 or 2 bytes) whole; here rank `rank` of `world` keeps only its
// contiguous row range of both.  world = 1 reproduces the reference's behaviour, including exit(1) on failure.
#pragma once
#include <cstdio>
#include <cstdlib>
#include <string>
#include "../../include/w4a8_b200.h"

struct QMatShard {
    uint8_t *wq = nullptr;   // rows * IN / 2 bytes (device)
    void *sc = nullptr;      // rows * IN / 32 scales (device)
    int64_t row0 = 0, rows = 0;
};

static inline QMatShard mat_shard(const std::string &dir, const std::string &name, size_t OUT, size_t IN, int scale_dtype,
                                  int rank, int world) {
    w4a8_qmat m;
    const std::string q4 = dir + "/" + name + "_q4.bin", sc = dir + "/" + name + "_scale.bin";
    if (w4a8_load_qmat_shard(q4.c_str(), sc.c_str(), (int64_t)OUT, (int64_t)IN, scale_dtype, rank, world, &m) != W4A8_OK) {
        fprintf(stderr, "w4a8 loader: %s\n", w4a8_last_error());
        exit(1);
    }
    QMatShard r;
    r.wq = m.wq; r.sc = m.sc; r.row0 = m.row0; r.rows = m.rows;
    return r;
}
