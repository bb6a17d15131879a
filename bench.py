#!/usr/bin/env python
"""Benchmark of the W4A8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Headline metric: HBM throughput of the W4A8 decode GEMV at M=1 on the
Qwen3.5-27B-class MLP up/gate shape K=5120, N=17408 (benchmark configuration 2 of 5); one step = one GEMV launch
through the C ABI over the next of several distinct weight copies (more bytes than the 126 MB L2, so every
step streams its weights from HBM).  `value` = algorithmic bytes / time with all inputs resident in HBM;
`e2e` = the same product through w4a8_linear (quantize + GEMV) with HOST activations and outputs, the
host<->device copies inside the timed region.  The M=2..16 sweep and the M=2048 prefill GEMM (quantize_x
included) are reported in `extra`.  At N > 1 the weights are sharded along N (rows of Wq), every rank
computes its slice and an NCCL all-gather reassembles Y (strong scaling: the total matrix is fixed).

--impl reference times the CPU restatement of the reference path (oracle/, all host threads) on bounded
samples of the same workload: the reference has no CPU build of its own and its CUDA kernels are reported,
rebuilt for sm_100a, inside the default arm's `extra.reference_kernels_sm100a`.
"""
import argparse
import ctypes
import importlib
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
K_DIM, N_DIM = 5120, 17408
L2_BYTES = 126 * 1024 * 1024
NCU_TRAFFIC = {  # dram__bytes_read.sum + dram__bytes_write.sum per launch, from one ncu capture of each kernel
    "gemv_m1": 55.77e6,   # the dp4a streaming kernel, M=1, K=5120, N=17408
}
# One string for both arms (the driver compares the two arms' `config.workload`).
WORKLOAD = "W4A8 decode GEMV M=1 K=5120 N=17408, int4 group-32 weights + fp32 scales (benchmark configuration 2 of 5)"
MIN_TIMED_MS = 20.0       # every timed leg replays its steps until at least this much device time is covered


def load_package():
    name = "dgx_serving_b200"
    if name in sys.modules:
        return sys.modules[name]
    path = os.path.join(ROOT, "dgx-serving_b200", "__init__.py")
    spec = importlib.util.spec_from_file_location(name, path, submodule_search_locations=[os.path.dirname(path)])
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def load_oracle():
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    oracle.lib()
    return oracle


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    return 6650.0, 1400.0, "fallback"


def host_cores():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except (AttributeError, OSError):
        return max(1, os.cpu_count() or 1)


def gemv_bytes(M, N, K, scale_bytes=4):
    """Algorithmic bytes of one GEMV launch: packed weights + scales + xq + xs + Y."""
    nb = K // 32
    return N * K // 2 + N * nb * scale_bytes + M * K + M * nb * 4 + M * N * 4


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm = [float(r[0]) for r in self.rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if r[1].replace(".", "").isdigit()]
        reasons = []
        for i, name in enumerate(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")):
            if any(r[3 + i].lower().startswith("active") for r in self.rows):
                reasons.append(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.rows)}


# ---------------------------------------------------------------------------------------------------------
def run_reference(args):
    """CPU restatement of the reference path on all host threads; bounded samples of the same workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    O = load_oracle()
    # all the cores this process may run on: torch.distributed.run exports OMP_NUM_THREADS=1, which must not
    # decide how many threads the CPU arm gets
    cores = host_cores()
    O.set_threads(cores)
    Wq, sw = O.make_weights(N_DIM, K_DIM, seed=20260002)
    X = O.make_activations(1, K_DIM, seed=20260102)
    xq, xs, _ = O.quantize_x_q8(X)
    per_step = max(1, int(os.environ.get("W4A8_REF_GEMVS_PER_STEP", "8")))
    for _ in range(args.warmup):
        O.gemm_mmq_w4a8(xq, xs, Wq, sw)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        for _ in range(per_step):
            O.gemm_mmq_w4a8(xq, xs, Wq, sw)
    dt = time.perf_counter() - t0
    launches = args.steps * per_step
    gbps = gemv_bytes(1, N_DIM, K_DIM) * launches / dt / 1e9
    line = {
        "impl": "reference", "metric": "w4a8_gemv_m1_hbm_gbps", "value": gbps, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "i8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": "%d GEMVs per step" % per_step},
        "cpu_baseline": {"value": gbps, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "%d scalar-C GEMVs of the full shape (oracle/w4a8_oracle.c, OpenMP)" % launches},
        "e2e": {"value": gbps, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the library has no CPU path (use --impl reference for the CPU arm)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    w = load_package()
    w.lib()
    sharded = importlib.import_module("dgx_serving_b200.sharded")
    hbm_peak, bf16_peak, peak_kind = measured_peaks()

    K, N = K_DIM, N_DIM
    nb = K // 32
    plan = sharded.shard_plan(N, world, w.shard_rows)
    row0, rows = plan[rank]
    shard_bytes = rows * (K // 2 + nb * 4)
    nbuf = max(3, int(np.ceil(2.2 * L2_BYTES / shard_bytes)))
    g = torch.Generator(device=dev)
    g.manual_seed(20260002 + rank)
    Wqs = [torch.randint(0, 256, (rows, K // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(nbuf)]
    sws = [(torch.randn(rows, nb, device=dev, generator=g).abs() * (0.02 / 7.0)) for _ in range(nbuf)]
    rng = np.random.default_rng(20260102)

    def make_x(M, outliers=False):
        X = rng.normal(0.0, 1.0, size=(M, K)).astype(np.float32)
        if outliers:
            X[rng.random(size=(M, K)) < 0.01] *= 20.0
        Xh = torch.from_numpy(X).pin_memory()
        Xd = Xh.to(dev)
        xq = torch.empty((M, K), dtype=torch.int8, device=dev)
        xs = torch.empty((M, nb), dtype=torch.float32, device=dev)
        xsum = torch.empty((M, nb), dtype=torch.int32, device=dev)
        w.launch_quantize_x_q8(Xd, xq, xs, xsum, K, M)
        torch.cuda.synchronize()
        return Xh, Xd, xq, xs, xsum

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return float(t.item())
        return ms

    timing_log = {}

    def time_steps(step_fn, steps, warmup, graph, after_fn=None, tag=None, min_ms=None):
        """step_fn(i, stream_handle) enqueues one step; after_fn(n, stream_handle), if given, is enqueued after every
        block of n steps (eager warm-up block, and as the last node of the captured graph).  One block = `steps` steps
        (a CUDA graph of them, or an eager loop); blocks are replayed back to back, each between its own pair of CUDA
        events on the launching stream, until at least `min_ms` of device time is covered.  Returns the MEDIAN block time
        in ms (max over ranks); the minimum and the number of blocks go to timing_log[tag]."""
        min_ms = args.min_timed_ms if min_ms is None else min(min_ms, args.min_timed_ms)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            nw = max(warmup, 3)
            for i in range(nw):
                step_fn(i, s.cuda_stream)
            if after_fn:
                after_fn(nw, s.cuda_stream)
            torch.cuda.synchronize()
            gr = None
            if graph:
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=s):
                    for i in range(steps):
                        step_fn(i, s.cuda_stream)
                    if after_fn:
                        after_fn(steps, s.cuda_stream)

            def block():
                if gr is not None:
                    gr.replay()
                else:
                    for i in range(steps):
                        step_fn(i, s.cuda_stream)
                    if after_fn:
                        after_fn(steps, s.cuda_stream)
            block()                  # one untimed block: graph upload, clocks up
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            block()
            e1.record(s)
            torch.cuda.synchronize()
            est = max_over_ranks(e0.elapsed_time(e1))
            reps = int(min(400, max(3, np.ceil(min_ms / max(est, 1e-3)))))
            barrier()
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
            evs[0].record(s)
            for r in range(reps):
                block()
                evs[r + 1].record(s)
            torch.cuda.synchronize()
            barrier()
        times = [evs[r].elapsed_time(evs[r + 1]) for r in range(reps)]
        med, mn = max_over_ranks(float(np.median(times))), max_over_ranks(float(np.min(times)))
        if tag:
            timing_log[tag] = {"blocks": reps, "steps_per_block": steps, "ms_per_step_median": med / steps, "ms_per_step_min": mn / steps}
        return med

    # ---- headline: GEMV M=1 (N-sharded + all-gather when world > 1) -------------------------------------
    def gemv_case(M, steps, warmup, mode="fused", tag=None):
        """One step = the rank-local GEMV plus (world > 1) the exchange that leaves the whole Y[M, N] on every rank:
        mode "fused": peer stores from the GEMV epilogue + flag wait (w4a8_gemv_allgather / w4a8_allgather_wait);
        mode "nccl":  GEMV into a local slice, then an NCCL all-gather."""
        Xh, Xd, xq, xs, xsum = make_x(M)
        Yloc = torch.empty((M, rows), dtype=torch.float32, device=dev)
        after = None
        check = None
        # consecutive steps alternate between two Y buffers: a block of an odd number of steps is captured twice over, so
        # that the last step of one replay and the first of the next never share a buffer
        blk = steps if (steps % 2 == 0 or not (world > 1 and mode == "fused")) else 2 * steps
        if world > 1 and mode == "fused":
            ystride = (M * N * 4 + 255) // 256 * 256
            arena = w.Arena(2 * ystride, rank, world)
            handles = [None] * world
            dist.all_gather_object(handles, arena.export_handle())
            arena.connect_handles(handles)
            dist.barrier()

            def step(i, st):
                # one call: the rank-local GEMV, the push of its slice to every peer, and the wait for every peer's slice
                arena.gemv_allgather_sync(xq, xs, Wqs[i % nbuf], sws[i % nbuf], (i % 2) * ystride, K, rows, row0, N, M, 0, i + 1, 2000000, st)

            def after(n, st):
                arena.advance_epoch(n, st)
        else:
            def step(i, st):
                w.launch_gemv_w4a8_sb(xq, xs, Wqs[i % nbuf], sws[i % nbuf], Yloc, K, rows, M, 0, st)
                if world > 1:
                    sharded.all_gather_columns(Yloc, plan)     # NCCL all-gather -> Y[M, N] on every rank
        ms = time_steps(step, blk, warmup, graph=(world == 1 or mode == "fused"), after_fn=after, tag=tag) * steps / blk
        if world > 1 and mode == "fused":
            w.device_status()
            barrier()
            # outside the timed region: one more fused step, its gathered Y compared bit for bit with the NCCL path's
            st0 = torch.cuda.current_stream().cuda_stream
            arena.gemv_allgather_sync(xq, xs, Wqs[0], sws[0], 0, K, rows, row0, N, M, 0, 1, 2000000, st0)
            arena.advance_epoch(1, st0)
            w.launch_gemv_w4a8_sb(xq, xs, Wqs[0], sws[0], Yloc, K, rows, M, 0, st0)
            Yn = sharded.all_gather_columns(Yloc, plan)
            torch.cuda.synchronize()
            w.device_status()
            same = bool(torch.equal(arena.tensor(0, (M, N)), Yn.reshape(M, N)))
            t = torch.tensor([1 if same else 0], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MIN)
            check = "bitwise equal to the NCCL all-gather path on every rank" if int(t.item()) == 1 else "MISMATCH against the NCCL path"
            barrier()
            arena.close()
        total_bytes = gemv_bytes(M, N, K)          # all ranks together stream the whole matrix once per step
        return ms, total_bytes * steps / (ms * 1e-3) / 1e9, (Xh, Xd, xq, xs, xsum), check

    sampler = ClockSampler(local) if rank == 0 else None
    ms, gbps, xin, gather_check = gemv_case(1, args.steps, args.warmup, tag="headline")
    clocks = sampler.stop() if sampler else None

    # kernel-only time of this rank's GEMV (no collective), for the roofline of the dominant kernel
    Xh, Xd, xq, xs, xsum = xin
    Yloc = torch.empty((1, rows), dtype=torch.float32, device=dev)
    ms_k = time_steps(lambda i, st: w.launch_gemv_w4a8_sb(xq, xs, Wqs[i % nbuf], sws[i % nbuf], Yloc, K, rows, 1, 0, st),
                      args.steps, args.warmup, graph=True, tag="kernel_only")
    per_launch_us = ms_k * 1e3 / args.steps
    achieved = gemv_bytes(1, rows, K) / (per_launch_us * 1e-6) / 1e9

    # ---- e2e: host fp32 activations in, host fp32 outputs back, through w4a8_linear ------------------------
    e2e_steps = max(10, min(args.steps, 200))
    if world == 1:
        Yh = torch.empty((1, rows), dtype=torch.float32).pin_memory()

        def e2e_step(i, st):
            # one C-ABI call: H2D of X, quantize_x + GEMV, D2H of Y, stream synchronise (the caller reads Y on the host)
            w.linear_host(Xh, Yh, Xd, xq, xs, xsum, Yloc, Wqs[i % nbuf], sws[i % nbuf], 1, rows, K, 0, st)
        ms_e = time_steps(e2e_step, e2e_steps, 3, graph=False, tag="e2e")
        e2e_path = "w4a8_linear_host: pinned host X -> quantize_x + gemv -> pinned host Y, one C-ABI call per step"
    else:
        # sharded: host X in on every rank, quantize_x, the rank's GEMV with the fused exchange, and the WHOLE gathered
        # Y[1, N] back to the host on every rank; stream synchronised every step
        Yh = torch.empty((1, N), dtype=torch.float32).pin_memory()
        estride = (N * 4 + 255) // 256 * 256
        earena = w.Arena(2 * estride, rank, world)
        ehandles = [None] * world
        dist.all_gather_object(ehandles, earena.export_handle())
        earena.connect_handles(ehandles)
        dist.barrier()
        ecount = [0]

        def e2e_step(i, st):
            ecount[0] += 1
            ts = torch.cuda.current_stream()
            Xd.copy_(Xh, non_blocking=True)
            w.launch_quantize_x_q8(Xd, xq, xs, xsum, K, 1, st)
            off = (ecount[0] % 2) * estride
            earena.gemv_allgather_sync(xq, xs, Wqs[i % nbuf], sws[i % nbuf], off, K, rows, row0, N, 1, 0, ecount[0], 2000000, st)
            Yh.copy_(earena.tensor(off, (1, N)), non_blocking=True)
            ts.synchronize()
        ms_e = time_steps(e2e_step, e2e_steps, 3, graph=False, tag="e2e")
        w.device_status()
        barrier()
        earena.close()
        e2e_path = ("pinned host X -> H2D -> quantize_x -> w4a8_gemv_allgather_sync (rank's rows, slice pushed to every peer, wait for "
                    "every peer) -> D2H of the whole gathered Y[1, N] -> stream synchronise, on every rank")
    e2e_gbps = gemv_bytes(1, N, K) * e2e_steps / (ms_e * 1e-3) / 1e9

    extra = {}
    if world > 1:
        ms_n, gb_n, _, _ = gemv_case(1, args.steps, args.warmup, mode="nccl")
        extra["nccl_allgather_path"] = {"ms_per_step": ms_n / args.steps, "gbps": gb_n}
        extra["fused_allgather_check_m1"] = gather_check
        extra["rank_local_kernel_us"] = per_launch_us
        sw_ = {}
        for M in (8, 16):
            ms_m, gb_m, _, chk = gemv_case(M, max(20, args.steps // 2), 3)
            sw_[str(M)] = {"us": ms_m * 1e3 / max(20, args.steps // 2), "gbps": gb_m, "check": chk}
        extra["gemv_sweep_fused_allgather"] = sw_
        # ---- N-sharded prefill GEMM M=2048: quantize_x + GEMM on the rank's rows; Y[M, N] complete on every rank either by
        # peer stores from the GEMM epilogue + flag wait (w4a8_gemm_allgather) or by an NCCL all-gather of the slices ----------
        Mg = 2048
        Xh2, Xd2, xq2, xs2, xsum2 = make_x(Mg, outliers=True)
        Yl2 = torch.empty((Mg, rows), dtype=torch.float32, device=dev)
        gstride = (Mg * N * 4 + 255) // 256 * 256
        garena = w.Arena(2 * gstride, rank, world)
        ghandles = [None] * world
        dist.all_gather_object(ghandles, garena.export_handle())
        garena.connect_handles(ghandles)
        dist.barrier()
        gepoch = [0]

        def gemm_fused(i, st):
            gepoch[0] += 1
            w.launch_quantize_x_q8(Xd2, xq2, xs2, xsum2, K, Mg, st)
            garena.gemm_allgather_sync(xq2, xs2, Wqs[i % nbuf], sws[i % nbuf], (gepoch[0] % 2) * gstride, Mg, rows, row0, N, K, 0, gepoch[0], 5000000, st)

        def gemm_nccl(i, st):
            w.linear(Xd2, xq2, xs2, xsum2, Wqs[i % nbuf], sws[i % nbuf], Yl2, Mg, rows, K, 0, 0, st)
            sharded.all_gather_columns(Yl2, plan)

        def gemm_local(i, st):
            w.linear(Xd2, xq2, xs2, xsum2, Wqs[i % nbuf], sws[i % nbuf], Yl2, Mg, rows, K, 0, 0, st)
        ms_gf = time_steps(gemm_fused, 5, 3, graph=False) / 5
        w.device_status()
        ms_g = time_steps(gemm_nccl, 5, 3, graph=False) / 5
        ms_gl = time_steps(gemm_local, 5, 3, graph=False) / 5
        w.device_status()
        barrier()
        garena.close()
        tops = lambda ms_: 2.0 * Mg * N * K / (ms_ * 1e-3) / 1e12
        extra["gemm_m2048_n_sharded"] = {"ms_per_step_fused_allgather": ms_gf, "int8_tops_whole_job_fused_allgather": tops(ms_gf),
                                         "ms_per_step_nccl_allgather": ms_g, "int8_tops_whole_job_nccl_allgather": tops(ms_g),
                                         "ms_rank_local_quantize_gemm": ms_gl, "int8_tops_without_allgather": tops(ms_gl)}
        del Yl2
        # ---- benchmark configuration 5 (128 experts, top-8) split over the ranks: 128 experts, 128 / world per GPU, top-8, M = 8 and 512 tokens; every
        # rank computes the slots routed to its experts, the slots' down outputs are exchanged through the arenas and every
        # rank combines (w4a8_moe_block_shard).  A CUDA graph of 10 blocks; its last node advances the arena's epoch base. ----
        if 128 % world == 0:
            E_, topk_, H_, MI_ = 128, 8, 2048, 768
            per_ = E_ // world
            gm = torch.Generator(device=dev); gm.manual_seed(77)                     # same routing and activations on every rank
            gu_w = torch.randint(0, 256, (per_, 2 * MI_, H_ // 2), dtype=torch.uint8, device=dev, generator=g)
            gu_s = torch.randn(per_, 2 * MI_, H_ // 32, device=dev, generator=g).abs() * (0.16 / 7.0)
            dn_w = torch.randint(0, 256, (per_, H_, MI_ // 2), dtype=torch.uint8, device=dev, generator=g)
            dn_s = torch.randn(per_, H_, MI_ // 32, device=dev, generator=g).abs() * (0.02 / 7.0)
            shard = {}
            for tok_ in (8, 512):
                n2_ = torch.randn(tok_, H_, device=dev, generator=gm)
                idx_ = torch.rand(tok_, E_, device=dev, generator=gm).argsort(dim=1)[:, :topk_].reshape(-1).to(torch.int32)
                dw_ = torch.rand(tok_ * topk_, device=dev, generator=gm)
                out_ = torch.empty((tok_, H_), dtype=torch.float32, device=dev)
                lay_ = w.moe_layout_for(tok_, topk_, H_, MI_, per_)
                ws_ = torch.empty(lay_.bytes, dtype=torch.uint8, device=dev)
                sstride = (tok_ * topk_ * H_ * 4 + 255) // 256 * 256
                marena = w.Arena(2 * sstride, rank, world)
                mh = [None] * world
                dist.all_gather_object(mh, marena.export_handle())
                marena.connect_handles(mh)
                dist.barrier()

                def moe_step(i, st):       # epochs are relative to the arena's base, which the last node of every block advances
                    w.moe_block_shard(n2_, gu_w, gu_s, dn_w, dn_s, idx_, dw_, out_, tok_, topk_, H_, MI_, rank * per_, per_, ws_, marena,
                                      (i % 2) * sstride, i + 1, 0, 0, 5000000, 0, st)
                nst = 10
                ms_ms = time_steps(moe_step, nst, 4, graph=True, after_fn=lambda n, st: marena.advance_epoch(n, st)) / nst
                w.device_status()
                barrier()
                marena.close()
                ops = 2.0 * tok_ * topk_ * (2 * MI_ * H_ + H_ * MI_)
                shard["m%d" % tok_] = {"us_per_block": ms_ms * 1e3, "experts_per_gpu": per_, "int8_tops_whole_job": ops / (ms_ms * 1e-3) / 1e12,
                                       "exchange_bytes_per_rank": tok_ * topk_ * H_ * 4 // world * (world - 1)}
            extra["moe_block_128e_top8_expert_sharded"] = shard
            del gu_w, gu_s, dn_w, dn_s
    if world == 1:
        # ---- sweep M = 2..16 on the same shape ------------------------------------------------------------
        sweep = {"1": {"us": per_launch_us, "gbps": achieved, "frac_of_measured_hbm": achieved / hbm_peak,
                       "frac_of_8tbs": achieved / 8000.0}}
        for M in (2, 4, 8, 16):
            ms_m, gb_m, _, _ = gemv_case(M, max(20, args.steps // 2), 3)
            us = ms_m * 1e3 / max(20, args.steps // 2)
            sweep[str(M)] = {"us": us, "gbps": gb_m, "frac_of_measured_hbm": gb_m / hbm_peak, "frac_of_8tbs": gb_m / 8000.0}
        extra["gemv_sweep_k5120_n17408"] = sweep
        # ---- prefill GEMM, quantize_x inside the timed region (benchmark configuration 4) ------------------------
        gemm, quant = {}, {}
        for M in (512, 2048, 8192):
            Xh2, Xd2, xq2, xs2, xsum2 = make_x(M, outliers=True)
            Y2 = torch.empty((M, N), dtype=torch.float32, device=dev)
            st_n = 5 if M < 8192 else 3
            ms_g = time_steps(lambda i, st: w.linear(Xd2, xq2, xs2, xsum2, Wqs[i % nbuf], sws[i % nbuf], Y2, M, N, K, 0, 0, st),
                              st_n, 3, graph=False)
            w.device_status()
            us = ms_g * 1e3 / st_n
            tops = 2.0 * M * N * K / (us * 1e-6) / 1e12
            gemm[str(M)] = {"us": us, "int8_tops": tops, "frac_of_nominal_4500": tops / 4500.0,
                            "frac_of_2x_measured_bf16": tops / (2.0 * bf16_peak)}
            del Y2
            if M >= 2048:
                # ---- quantize_x alone (HBM-bound, 5.25 bytes per element): rotating inputs larger than L2 -------------
                nx = max(2, int(np.ceil(1.5 * L2_BYTES / (M * K * 4.0))))
                Xs_ = [Xd2] + [torch.randn(M, K, device=dev, generator=g) for _ in range(nx - 1)]
                ms_q = time_steps(lambda i, st: w.launch_quantize_x_q8(Xs_[i % nx], xq2, xs2, xsum2, K, M, st), 20, 3, graph=True)
                us_q = ms_q * 1e3 / 20
                qb = 5.25 * M * K
                quant[str(M)] = {"us": us_q, "gbps": qb / (us_q * 1e-6) / 1e9, "frac_of_measured_hbm": qb / (us_q * 1e-6) / 1e9 / hbm_peak,
                                 "algorithmic_bytes": qb}
                del Xs_
        extra["gemm_quantize_included_k5120_n17408"] = gemm
        extra["quantize_x_k5120"] = quant
        # ---- fp16 weight scales (scale_dtype 1), M=1: 10 % fewer bytes per launch --------------------------------
        sws16 = [t.half() for t in sws]
        ms_h = time_steps(lambda i, st: w.launch_gemv_w4a8_sb(xq, xs, Wqs[i % nbuf], sws16[i % nbuf], Yloc, K, N, 1, 1, st),
                          args.steps, 3, graph=True)
        us_h = ms_h * 1e3 / args.steps
        extra["gemv_m1_fp16_scales"] = {"us": us_h, "gbps": gemv_bytes(1, N, K, 2) / (us_h * 1e-6) / 1e9}
        del sws16
        # ---- gate + up against one quantized row: two launches, or one w4a8_gemv_multi launch -------------------------
        Yg, Yu = torch.empty((1, N), dtype=torch.float32, device=dev), torch.empty((1, N), dtype=torch.float32, device=dev)

        def two_launches(i, st):
            w.launch_gemv_w4a8_sb(xq, xs, Wqs[(2 * i) % nbuf], sws[(2 * i) % nbuf], Yg, K, N, 1, 0, st)
            w.launch_gemv_w4a8_sb(xq, xs, Wqs[(2 * i + 1) % nbuf], sws[(2 * i + 1) % nbuf], Yu, K, N, 1, 0, st)

        def one_launch(i, st):
            a, b = (2 * i) % nbuf, (2 * i + 1) % nbuf
            w.gemv_multi(xq, xs, [Wqs[a], Wqs[b]], [sws[a], sws[b]], [Yg, Yu], [N, N], K, 1, 0, st)
        ns = max(20, args.steps // 2)
        us_two = time_steps(two_launches, ns, 3, graph=True) * 1e3 / ns
        us_one = time_steps(one_launch, ns, 3, graph=True) * 1e3 / ns
        extra["gate_up_pair_m1"] = {"us_two_launches": us_two, "us_one_launch": us_one,
                                    "gbps_one_launch": 2 * gemv_bytes(1, N, K) / (us_one * 1e-6) / 1e9}
        # ---- an lm_head-sized matrix (vocabulary 151936 x K=5120, 487 MB): auto policy streams it with bulk copies ----
        Nv = 151936
        vq = [torch.randint(0, 256, (Nv, K // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(2)]
        vs = [(torch.randn(Nv, nb, device=dev, generator=g).abs() * (0.02 / 7.0)) for _ in range(2)]
        Yv = torch.empty((1, Nv), dtype=torch.float32, device=dev)
        ms_v = time_steps(lambda i, st: w.launch_gemv_w4a8_sb(xq, xs, vq[i % 2], vs[i % 2], Yv, K, Nv, 1, 0, st), 20, 3, graph=True)
        us_v = ms_v * 1e3 / 20
        gb_v = gemv_bytes(1, Nv, K) / (us_v * 1e-6) / 1e9
        extra["gemv_m1_lm_head_k5120_n151936"] = {"us": us_v, "gbps": gb_v, "frac_of_measured_hbm": gb_v / hbm_peak}
        del vq, vs, Yv
        # ---- benchmark configuration 3: Gemma4-12B-class layer set at M=8, launched back to back --------------------------
        layer = [(3840, 4096), (3840, 3840), (3840, 15360), (3840, 15360), (15360, 3840)]
        reps = 5                                                     # 5 distinct layers' worth of weights (648 MB > L2)
        lw = [[(torch.randint(0, 256, (n_, k_ // 2), dtype=torch.uint8, device=dev, generator=g),
                torch.randn(n_, k_ // 32, device=dev, generator=g).abs() * (0.02 / 7.0)) for (k_, n_) in layer] for _ in range(reps)]
        lx = {}
        for k_ in (3840, 15360):
            X_ = torch.randn(8, k_, device=dev, generator=g)
            q_ = torch.empty((8, k_), dtype=torch.int8, device=dev); s_ = torch.empty((8, k_ // 32), dtype=torch.float32, device=dev)
            w.launch_quantize_x_q8(X_, q_, s_, None, k_, 8)
            lx[k_] = (q_, s_)
        ly = {n_: torch.empty((8, n_), dtype=torch.float32, device=dev) for (_, n_) in layer}

        def layer_step(i, st):
            for (k_, n_), (wq_, sw_) in zip(layer, lw[i % reps]):
                w.launch_gemv_w4a8_sb(lx[k_][0], lx[k_][1], wq_, sw_, ly[n_], k_, n_, 8, 0, st)
        ms_l = time_steps(layer_step, 20, 3, graph=True)
        lbytes = sum(gemv_bytes(8, n_, k_) for (k_, n_) in layer)
        extra["gemma4_12b_layer_set_m8"] = {"us_per_layer": ms_l * 1e3 / 20, "gbps": lbytes / (ms_l / 20 * 1e-3) / 1e9,
                                            "algorithmic_bytes_per_layer": lbytes}
        del lw
        # ---- benchmark configuration 5: 128 experts, top-8, M=8 tokens, gate/up 2048->768 and down 768->2048 -----------------
        E, topk, tok = 128, 8, 8
        idx = torch.rand(tok, E, device=dev, generator=g).argsort(dim=1)[:, :topk].reshape(-1).to(torch.int32)   # top-k distinct experts per token
        moe = {}
        for name, (k_, n_, per_slot) in {"gate_or_up": (2048, 768, 0), "down": (768, 2048, 1)}.items():
            nrow = tok * topk if per_slot else tok
            wq_ = [torch.randint(0, 256, (E * n_, k_ // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(2)]
            sw_ = [torch.randn(E * n_, k_ // 32, device=dev, generator=g).abs() * (0.02 / 7.0) for _ in range(2)]
            X_ = torch.randn(nrow, k_, device=dev, generator=g)
            q_ = torch.empty((nrow, k_), dtype=torch.int8, device=dev); s_ = torch.empty((nrow, k_ // 32), dtype=torch.float32, device=dev)
            w.launch_quantize_x_q8(X_, q_, s_, None, k_, nrow)
            y_ = torch.empty((tok * topk, n_), dtype=torch.float32, device=dev)
            ms_m = time_steps(lambda i, st: w.moe_gemv(q_, s_, wq_[i % 2], sw_[i % 2], idx, y_, tok * topk, topk, per_slot, n_, k_, E, 0, st),
                              50, 3, graph=True)
            touched = int(torch.unique(idx).numel())
            by = touched * (n_ * k_ // 2 + n_ * (k_ // 32) * 4)
            moe[name] = {"us": ms_m * 1e3 / 50, "experts_touched": touched, "gbps_weights": by / (ms_m / 50 * 1e-3) / 1e9}
        extra["moe_128e_top8_m8"] = moe
        # ---- the whole routed-expert block (quantize, gate|up, activation + quantize, down, combine) at M = 8 and 512 -----
        H_, MI_ = 2048, 768
        blk = {}
        gu_w = [torch.randint(0, 256, (E, 2 * MI_, H_ // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(2)]
        gu_s = [torch.randn(E, 2 * MI_, H_ // 32, device=dev, generator=g).abs() * (0.16 / 7.0) for _ in range(2)]
        dn_w = [torch.randint(0, 256, (E, H_, MI_ // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(2)]
        dn_s = [torch.randn(E, H_, MI_ // 32, device=dev, generator=g).abs() * (0.02 / 7.0) for _ in range(2)]
        per_expert = 2 * MI_ * (H_ // 2 + (H_ // 32) * 4) + H_ * (MI_ // 2 + (MI_ // 32) * 4)     # 2,949,120 B: gate+up+down, fp32 scales
        for tok_ in (8, 512):
            n2_ = torch.randn(tok_, H_, device=dev, generator=g)
            idx_ = torch.rand(tok_, E, device=dev, generator=g).argsort(dim=1)[:, :topk].reshape(-1).to(torch.int32)
            dw_ = torch.rand(tok_ * topk, device=dev, generator=g)
            out_ = torch.empty((tok_, H_), dtype=torch.float32, device=dev)
            lay_ = w.moe_layout_for(tok_, topk, H_, MI_, E)
            ws_ = torch.empty(lay_.bytes, dtype=torch.uint8, device=dev)
            nst = 20 if tok_ <= 64 else 6
            ms_b = time_steps(lambda i, st: w.moe_block(n2_, gu_w[i % 2], gu_s[i % 2], dn_w[i % 2], dn_s[i % 2], idx_, dw_, out_, tok_, topk, H_, MI_,
                                                        E, ws_, 0, 0, st), nst, 3, graph=True)
            us_b = ms_b * 1e3 / nst
            touched = int(torch.unique(idx_).numel())
            ops = 2.0 * tok_ * topk * (2 * MI_ * H_ + H_ * MI_)
            refp_ = os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so")
            us_ref = None
            if os.path.exists(refp_):       # the reference's own fused expert path (W4A32 arithmetic: the nearest reference code)
                rk = ctypes.CDLL(refp_)
                if hasattr(rk, "ref_moe_fused_block"):
                    P_ = lambda t: ctypes.c_void_p(t.data_ptr())
                    nsl = tok_ * topk
                    fgu = torch.empty((nsl, 2 * MI_), dtype=torch.float32, device=dev)
                    fhid = torch.empty((nsl, MI_), dtype=torch.float32, device=dev)
                    fso = torch.empty((nsl, H_), dtype=torch.float32, device=dev)
                    nr = 10 if tok_ <= 64 else 2
                    ms_r = time_steps(lambda i, st: rk.ref_moe_fused_block(P_(n2_), P_(gu_w[i % 2]), P_(gu_s[i % 2]), P_(dn_w[i % 2]), P_(dn_s[i % 2]),
                                                                           P_(idx_), P_(dw_), P_(fgu), P_(fhid), P_(fso), P_(out_), tok_, H_, MI_, topk,
                                                                           0, ctypes.c_void_p(st)), nr, 3, graph=True, min_ms=5.0)
                    us_ref = ms_r * 1e3 / nr
                    del fgu, fhid, fso
            blk["m%d" % tok_] = {"us": us_b, "reference_w4a32_fused_path_sm100a_us": us_ref,
                                 "experts_touched": touched, "weight_bytes": touched * per_expert,
                                 "gbps_weights": touched * per_expert / (us_b * 1e-6) / 1e9, "int8_tops": ops / (us_b * 1e-6) / 1e12,
                                 "kernel": "grouped GEMV per slot" if tok_ * topk <= 128 else "sorted grouped tcgen05 GEMM"}
        extra["moe_block_128e_top8"] = blk
        del gu_w, gu_s, dn_w, dn_s
        # ---- the reference's own kernels rebuilt for sm_100a, same buffers (not part of the library) -------
        refp = os.path.join(ROOT, "oracle", "_ref", "libref_kernels.so")
        if os.path.exists(refp):
            ref = ctypes.CDLL(refp)
            P = lambda t: ctypes.c_void_p(t.data_ptr())
            ms_r = time_steps(lambda i, st: ref.ref_gemv_w4a8_mlp2(P(xq), P(xs), P(xsum), P(Wqs[i % nbuf]), P(sws[i % nbuf]), P(Yloc),
                                                                  K, N, 1, 0, ctypes.c_void_p(st)), args.steps, 3, graph=True)
            us_r = ms_r * 1e3 / args.steps
            Xh2, Xd2, xq2, xs2, xsum2 = make_x(2048, outliers=True)
            Y2 = torch.empty((2048, N), dtype=torch.float32, device=dev)

            def ref_gemm(i, st):
                ref.ref_quantize_x_q8(P(Xd2), P(xq2), P(xs2), P(xsum2), K, 2048, ctypes.c_void_p(st))
                ref.ref_gemm_mmq_w4a8(P(xq2), P(xs2), P(Wqs[i % nbuf]), P(sws[i % nbuf]), P(Y2), 2048, N, K, 0, ctypes.c_void_p(st))
            ms_rg = time_steps(ref_gemm, 3, 3, graph=False)
            refk = {}
            # the reference's batched decode kernels on the same buffers (a6: SB for 2..15 rows, a8: gemm_batch<16>)
            for Mr in (2, 4, 8, 16):
                Xr_, Xdr_, xqr, xsr, xsumr = make_x(Mr)
                Yr = torch.empty((Mr, N), dtype=torch.float32, device=dev)
                ms_sb = time_steps(lambda i, st: ref.ref_gemv_w4a8_sb(P(xqr), P(xsr), P(Wqs[i % nbuf]), P(sws[i % nbuf]), P(Yr), K, N, Mr, 0,
                                                                      ctypes.c_void_p(st)), 20, 3, graph=True)
                refk["gemv_w4a8_sb_m%d" % Mr] = {"us": ms_sb * 1e3 / 20}
                if Mr == 16:
                    ms_gb = time_steps(lambda i, st: ref.ref_gemm_batch_w4a8(P(xqr), P(xsr), P(Wqs[i % nbuf]), P(sws[i % nbuf]), P(Yr), K, N, 16, 0,
                                                                             ctypes.c_void_p(st)), 20, 3, graph=True)
                    refk["gemm_batch_w4a8_m16"] = {"us": ms_gb * 1e3 / 20}
                del Yr
            # the tile variants the graphs actually call for prefill (a11: 256x64 template, a12: raster order 1), kernel only
            for nm, fn_ in (("gemm_mmq_tmpl_256x64_m2048", lambda i, st: ref.ref_gemm_mmq_256x64(P(xq2), P(xs2), P(Wqs[i % nbuf]), P(sws[i % nbuf]), P(Y2),
                                                                                               2048, N, K, 0, ctypes.c_void_p(st))),
                            ("gemm_mmq_raster1_m2048", lambda i, st: ref.ref_gemm_mmq_raster_w4a8(P(xq2), P(xs2), P(Wqs[i % nbuf]), P(sws[i % nbuf]), P(Y2),
                                                                                                 2048, N, K, 0, 1, 8, ctypes.c_void_p(st))),
                            ("gemm_mmq_128x128_m2048", lambda i, st: ref.ref_gemm_mmq_w4a8(P(xq2), P(xs2), P(Wqs[i % nbuf]), P(sws[i % nbuf]), P(Y2),
                                                                                          2048, N, K, 0, ctypes.c_void_p(st)))):
                ms_t = time_steps(fn_, 3, 3, graph=False)
                refk[nm] = {"us": ms_t * 1e3 / 3, "int8_tops": 2.0 * 2048 * N * K / (ms_t / 3 * 1e-3) / 1e12}
            ms_rq = time_steps(lambda i, st: ref.ref_quantize_x_q8(P(Xd2), P(xq2), P(xs2), P(xsum2), K, 2048, ctypes.c_void_p(st)), 20, 3, graph=True)
            refk["quantize_x_q8_m2048"] = {"us": ms_rq * 1e3 / 20, "gbps": 5.25 * 2048 * K / (ms_rq / 20 * 1e-3) / 1e9}
            # ---- quantize_x fused into its producer, against the reference's two kernels (decode, one row) -----------
            ref.ref_rmsnorm.restype = ctypes.c_int
            ref.ref_glu.restype = ctypes.c_int
            H, F = K, N
            xh = torch.randn(1, H, device=dev, generator=g); wn = torch.randn(H, device=dev, generator=g) * 0.1
            nrm = torch.empty(1, H, device=dev)
            gg = torch.randn(1, F, device=dev, generator=g); uu = torch.randn(1, F, device=dev, generator=g)
            act = torch.empty(1, F, device=dev)
            fq = torch.empty((1, F), dtype=torch.int8, device=dev); fs = torch.empty((1, F // 32), dtype=torch.float32, device=dev)
            fsum = torch.empty((1, F // 32), dtype=torch.int32, device=dev)

            def ref_norm_q(i, st):
                ref.ref_rmsnorm(P(xh), P(wn), P(nrm), 1, H, ctypes.c_float(1e-6), 1, ctypes.c_void_p(st))
                ref.ref_quantize_x_q8(P(nrm), P(fq), P(fs), P(fsum), H, 1, ctypes.c_void_p(st))

            def ref_glu_q(i, st):
                ref.ref_glu(P(gg), P(uu), P(act), ctypes.c_long(F), 0, ctypes.c_void_p(st))
                ref.ref_quantize_x_q8(P(act), P(fq), P(fs), P(fsum), F, 1, ctypes.c_void_p(st))
            fused = {}
            for name, ours, theirs in (
                    ("rmsnorm_zc+quantize_h5120", lambda i, st: w.launch_rmsnorm_quantize_x_q8(xh, wn, 1e-6, 1, None, fq, fs, fsum, H, 1, st), ref_norm_q),
                    ("swiglu+quantize_f17408", lambda i, st: w.launch_glu_quantize_x_q8(gg, uu, 0, None, fq, fs, fsum, F, 1, st), ref_glu_q)):
                us_o = time_steps(ours, 100, 3, graph=True) * 1e3 / 100
                us_t = time_steps(theirs, 100, 3, graph=True) * 1e3 / 100
                fused[name] = {"us_fused": us_o, "us_reference_two_kernels": us_t}
            extra["fused_quantize_m1"] = fused
            refk["gemv_w4a8_mlp2_m1"] = {"us": us_r, "gbps": gemv_bytes(1, N, K) / (us_r * 1e-6) / 1e9}
            refk["quantize+gemm_mmq_m2048"] = {"us": ms_rg * 1e3 / 3, "int8_tops": 2.0 * 2048 * N * K / (ms_rg / 3 * 1e-3) / 1e12}
            extra["reference_kernels_sm100a"] = refk
            del Y2

    cpu_baseline = None
    if world == 1:
        O = load_oracle()
        cores = host_cores()
        O.set_threads(cores)
        Wq_h, sw_h = Wqs[0].cpu().numpy(), sws[0].cpu().numpy()
        xq_h, xs_h = xq.cpu().numpy(), xs.cpu().numpy()
        O.gemm_mmq_w4a8(xq_h, xs_h, Wq_h, sw_h)
        n, t0 = 0, time.perf_counter()
        while time.perf_counter() - t0 < 10.0:
            O.gemm_mmq_w4a8(xq_h, xs_h, Wq_h, sw_h)
            n += 1
        dt = time.perf_counter() - t0
        cpu_baseline = {"value": gemv_bytes(1, N, K) * n / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                        "sample": "%d scalar-C GEMVs of the full M=1 shape in %.1f s (oracle/w4a8_oracle.c, OpenMP)" % (n, dt)}

    if rank == 0:
        line = {
            "metric": "w4a8_gemv_m1_hbm_gbps", "value": gbps, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "i8", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "parallelism": ("n-shard x%d, all-gather fused into the GEMV (every output also goes to every peer as an 8-byte {value, epoch tag} store over NVLink; the same launch polls the peers' slots)" % world)
                       if world > 1 else "single GPU",
                       "l2": "rotating %d distinct weight copies per rank (%.0f MB > 126 MB L2)" % (nbuf, nbuf * shard_bytes / 1e6),
                       "launch": "CUDA graph of %d steps, replayed %d times (>= %.0f ms timed); value from the median replay, min in `timing`"
                                 % (timing_log["headline"]["steps_per_block"], timing_log["headline"]["blocks"], args.min_timed_ms)},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": NCU_TRAFFIC["gemv_m1"] if world == 1 else None, "peak_kind": "of " + peak_kind,
                         "kernel": "gemv_w4a8_dp4a_kernel (w4a8_gemv, M=1, auto policy), rank-local slice of %d rows" % rows, "us_per_launch": per_launch_us,
                         "algorithmic_bytes_per_launch": gemv_bytes(1, rows, K), "frac_of_nominal_8tbs": achieved / 8000.0},
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": e2e_gbps, "unit": "GB/s", "h2d_bytes_per_step": K * 4, "d2h_bytes_per_step": (rows if world == 1 else N) * 4,
                    "ms_per_step": ms_e / e2e_steps, "path": e2e_path},
            "gpu_launches": args.steps,
            "timing": {k: timing_log[k] for k in ("headline", "kernel_only", "e2e") if k in timing_log},
            "clocks": clocks,
            "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_kernel_case(args):
    """Small single-kernel run for profiler captures: `--kernel-case gemv_m1 | gemv_m8 | gemv_m16 | gemm_m512 | quantize_m2048 |
    moe_m512 | moe_m8` launches that kernel (moe: the routed-expert block of benchmark configuration 5 (128 experts, top-8), all of its kernels)
    `--steps` times (eagerly, no graph) over 3 rotating copies of the K=5120 x N=17408 weights (167 MB, larger than L2,
    well under 1 GB on the device; moe: one 378 MB set of 128 experts) and prints its CUDA-event time.  Not a bench line."""
    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = load_package()
    w.lib()
    name = args.kernel_case
    kind, M = name.split("_m")
    M = int(M)
    K, N, nb = K_DIM, N_DIM, K_DIM // 32
    g = torch.Generator(device=dev)
    g.manual_seed(20260003)
    Wqs = [torch.randint(0, 256, (N, K // 2), dtype=torch.uint8, device=dev, generator=g) for _ in range(3)]
    sws = [(torch.randn(N, nb, device=dev, generator=g).abs() * (0.02 / 7.0)) for _ in range(3)]
    X = torch.randn(M, K, device=dev, generator=g)
    xq = torch.empty((M, K), dtype=torch.int8, device=dev)
    xs = torch.empty((M, nb), dtype=torch.float32, device=dev)
    xsum = torch.empty((M, nb), dtype=torch.int32, device=dev)
    w.launch_quantize_x_q8(X, xq, xs, xsum, K, M)
    Y = torch.empty((M, N), dtype=torch.float32, device=dev)
    s = torch.cuda.Stream()
    steps = max(1, min(args.steps, 20))
    if kind == "moe":
        del Wqs, sws
        E, topk, H_, MI_ = 128, 8, 2048, 768
        gu_w = torch.randint(0, 256, (E, 2 * MI_, H_ // 2), dtype=torch.uint8, device=dev, generator=g)
        gu_s = torch.randn(E, 2 * MI_, H_ // 32, device=dev, generator=g).abs() * (0.16 / 7.0)
        dn_w = torch.randint(0, 256, (E, H_, MI_ // 2), dtype=torch.uint8, device=dev, generator=g)
        dn_s = torch.randn(E, H_, MI_ // 32, device=dev, generator=g).abs() * (0.02 / 7.0)
        n2 = torch.randn(M, H_, device=dev, generator=g)
        idx = torch.rand(M, E, device=dev, generator=g).argsort(dim=1)[:, :topk].reshape(-1).to(torch.int32)
        dw = torch.rand(M * topk, device=dev, generator=g)
        out = torch.empty((M, H_), dtype=torch.float32, device=dev)
        ws = torch.empty(w.moe_layout_for(M, topk, H_, MI_, E).bytes, dtype=torch.uint8, device=dev)

    def launch(i):
        if kind == "moe":
            w.moe_block(n2, gu_w, gu_s, dn_w, dn_s, idx, dw, out, M, topk, H_, MI_, E, ws, 0, 0, s.cuda_stream)
        elif kind == "quantize":
            w.launch_quantize_x_q8(X, xq, xs, xsum, K, M, s.cuda_stream)
        elif kind == "gemv":
            w.launch_gemv_w4a8_sb(xq, xs, Wqs[i % 3], sws[i % 3], Y, K, N, M, 0, s.cuda_stream)
        elif kind == "gemm":
            w.launch_gemm_mmq_w4a8(xq, xs, Wqs[i % 3], sws[i % 3], Y, M, N, K, 0, s.cuda_stream)
        else:
            raise SystemExit("unknown kernel case " + name)
    with torch.cuda.stream(s):
        for i in range(3):
            launch(i)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        for i in range(steps):
            launch(i)
        e1.record(s)
        torch.cuda.synchronize()
    w.device_status()
    print(json.dumps({"kernel_case": name, "launches": steps, "us_per_launch": e0.elapsed_time(e1) * 1e3 / steps}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel-case", default=None,
                    help="profiler helper: gemv_m1, gemv_m8, gemv_m16, gemm_m512, quantize_m2048, moe_m8 or moe_m512 (see run_kernel_case)")
    ap.add_argument("--min-timed-ms", type=float, default=MIN_TIMED_MS,
                    help="every timed leg replays its block of steps until this much device time is covered (at least 3 blocks); "
                         "0 keeps a profiler's launch list short")
    args = ap.parse_args()
    if args.kernel_case:
        run_kernel_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
