"""CPU tests of the C-ABI boundary and the host logic (no compute call needs a GPU).

  - libw4a8_b200.so loads and exports every function include/w4a8_b200.h declares;
  - argument validation that happens before any device work returns the documented status codes;
  - the row-shard arithmetic; the N-sharded all-gather plumbing with 2 gloo ranks on CPU.
"""
import ctypes
import os
import re
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "w4a8_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(w4a8_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(w4a8):
    lib = w4a8.lib()
    names = declared_functions()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), "missing export " + n
    assert set(names) == set(w4a8.EXPORTS), (set(names) ^ set(w4a8.EXPORTS))
    assert lib.w4a8_version() >= 100
    # nothing but the declared C ABI (and no oracle symbol) is exported
    out = subprocess.run(["nm", "-D", "--defined-only", w4a8.LIB_PATH], capture_output=True, text=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if " T " in l}
    assert {e for e in exported if e.startswith("w4a8_")} == set(names)
    assert not [e for e in exported if "oracle" in e]


def test_argument_validation_before_any_device_work(w4a8):
    lib = w4a8.lib()
    p = ctypes.c_void_p(4096)
    assert lib.w4a8_quantize_x_q8(p, p, p, p, 100, 1, None) == w4a8.ERR_ARG          # IN % 32 != 0
    assert b"multiple of 32" in lib.w4a8_last_error()
    assert lib.w4a8_quantize_x_q8(p, p, p, p, 64, 0, None) == w4a8.OK                # empty input: nothing to do
    assert lib.w4a8_quantize_x_q8(None, p, p, p, 64, 1, None) == w4a8.ERR_ARG
    assert lib.w4a8_gemv(p, p, p, p, p, 64, 0, 1, 0, None) == w4a8.OK                # OUT = 0
    assert lib.w4a8_gemv(p, p, None, p, p, 64, 8, 1, 0, None) == w4a8.ERR_ARG
    assert lib.w4a8_gemv(p, p, p, p, p, 48, 8, 1, 0, None) == w4a8.ERR_ARG           # K % 32
    assert lib.w4a8_gemv(p, p, p, p, p, 64, 8, 1, 7, None) == w4a8.ERR_ARG           # scale_dtype
    assert lib.w4a8_gemm(p, p, p, p, p, 0, 8, 64, 0, None) == w4a8.OK                # M = 0 (kernels/gemm_mmq_raster.cuh:118)
    assert lib.w4a8_gemm(p, p, p, p, p, -1, 8, 64, 0, None) == w4a8.ERR_ARG
    assert lib.w4a8_gemm(ctypes.c_void_p(4100), p, p, p, p, 4, 8, 64, 0, None) == w4a8.ERR_ALIGN   # TMA needs 16 B
    assert lib.w4a8_group_dots(p, p, p, 4, 8, 64, 9, None) in (w4a8.ERR_ARG, w4a8.ERR_CUDA, w4a8.ERR_UNSUPPORTED)
    assert lib.w4a8_moe_gemv(p, p, p, p, None, p, 4, 2, 0, 8, 64, 4, 0, None) == w4a8.ERR_ARG
    assert lib.w4a8_gemm_splitk_workspace_bytes(16, 256, 1024, 4) == 4 * 16 * 256 * 4
    assert lib.w4a8_gemm_splitk_workspace_bytes(16, 17408, 5120, 0) == 0                           # 136 tiles: no split
    assert lib.w4a8_gemm_splitk_workspace_bytes(16, 256, 1024, 2 ** 31 - 1) == 0                   # absurd split count
    assert lib.w4a8_gemm_splitk(p, p, p, p, p, 16, 256, 1024, 0, 2 ** 31 - 1, p, 1 << 20, None) == w4a8.ERR_ARG
    assert lib.w4a8_gemm_splitk_static(p, p, p, p, p, 16, 256, 1024, 0, 2 ** 31 - 1, None) == w4a8.ERR_ARG
    # routed-expert block: shapes and workspace are checked before any device work
    z = ctypes.c_size_t(1 << 30)
    assert lib.w4a8_moe_block(p, p, p, p, p, p, p, p, 4, 2, 48, 32, 4, 0, 0, p, z, None) == w4a8.ERR_ARG      # H % 32
    assert lib.w4a8_moe_block(p, p, p, p, p, p, p, p, 4, 2, 64, 32, 4, 0, 3, p, z, None) == w4a8.ERR_ARG      # activation
    assert lib.w4a8_moe_block(p, p, p, p, p, p, p, p, 4, 2, 64, 32, 4000, 0, 0, p, z, None) == w4a8.ERR_ARG   # experts > 1024
    assert lib.w4a8_moe_block(p, p, p, p, p, None, p, p, 4, 2, 64, 32, 4, 0, 0, p, z, None) == w4a8.ERR_ARG   # no routing indices
    assert lib.w4a8_moe_block(p, p, p, p, p, p, p, p, 4, 2, 64, 32, 4, 0, 0, p, ctypes.c_size_t(64), None) == w4a8.ERR_ARG
    assert b"workspace" in lib.w4a8_last_error()
    assert lib.w4a8_moe_block(p, p, p, p, p, p, p, p, 0, 2, 64, 32, 4, 0, 0, p, z, None) == w4a8.OK           # no tokens


def test_moe_layout_is_disjoint_and_aligned(w4a8):
    S, topk, H, MI, E = 512, 8, 2048, 768, 128
    lay = w4a8.moe_layout_for(S, topk, H, MI, E)
    n = S * topk
    sizes = {"perm": n * 4, "pos": n * 4, "offsets": (E + 1) * 4, "items": (E + n // 64 + 1) * 16, "num_items": 4, "xq": S * H,
             "xs": S * (H // 32) * 4, "xq_g": n * H, "xs_g": n * (H // 32) * 4, "gu": n * 2 * MI * 4, "xq_h": n * MI, "xs_h": n * (MI // 32) * 4,
             "sout": n * H * 4}
    spans = sorted((getattr(lay, k), getattr(lay, k) + v) for k, v in sizes.items())
    assert all(a % 256 == 0 for a, _ in spans)
    assert all(spans[i][1] <= spans[i + 1][0] for i in range(len(spans) - 1))
    assert spans[-1][1] <= lay.bytes
    with pytest.raises(w4a8.W4A8Error):
        w4a8.moe_layout_for(4, 2, 64, 32, 5000)


def test_no_cpu_fallback_without_a_device(w4a8):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    lib = w4a8.lib()
    p = ctypes.c_void_p(4096)
    rc = lib.w4a8_gemv(p, p, p, p, p, 64, 8, 1, 0, None)
    assert rc in (w4a8.ERR_CUDA, w4a8.ERR_UNSUPPORTED)                                              # fails loudly
    assert lib.w4a8_last_error() != b""


@pytest.mark.parametrize("N,world", [(17408, 1), (17408, 2), (17408, 8), (3840, 8), (1001, 8), (5, 8), (0, 4)])
def test_shard_rows_partition(w4a8, N, world):
    plan = [w4a8.shard_rows(N, r, world) for r in range(world)]
    assert plan[0][0] == 0
    assert sum(r for _, r in plan) == N
    for (a0, a), (b0, _) in zip(plan, plan[1:]):
        assert a0 + a == b0
    sizes = [r for _, r in plan]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes)      # remainder goes to the last ranks
    with pytest.raises(w4a8.W4A8Error):
        w4a8.shard_rows(N, world, world)


def test_loader_rejects_short_files_before_touching_a_device(w4a8, tmp_path):
    q4, sc = tmp_path / "a_q4.bin", tmp_path / "a_scale.bin"
    q4.write_bytes(b"\x88" * 100)
    sc.write_bytes(b"\x00" * 8)
    with pytest.raises(w4a8.W4A8Error) as ei:
        w4a8.load_qmat_shard(str(q4), str(sc), 64, 64, 0, 0, 1)         # needs 2048 + 512 bytes
    assert ei.value.code == w4a8.ERR_IO
    with pytest.raises(w4a8.W4A8Error) as ei:
        w4a8.load_qmat_shard(str(tmp_path / "missing.bin"), str(sc), 64, 64, 0, 0, 1)
    assert ei.value.code == w4a8.ERR_IO


_WORKER = r'''
import os, sys
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, os.path.join(ROOT, "oracle"))
import numpy as np, torch, torch.distributed as dist
from conftest import load_package
import oracle as O
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
w = load_package()
import importlib
sharded = importlib.import_module("dgx_serving_b200.sharded")
for (M, N, K) in [(1, 64, 128), (5, 64, 128), (3, 37, 96)]:
    Wq, sw = O.make_weights(N, K, seed=1)
    X = O.make_activations(M, K, seed=2)
    def compute(Xt, row0, rows):
        xq, xs, _ = O.quantize_x_q8(Xt.numpy())
        return torch.from_numpy(O.gemm_mmq_w4a8(xq, xs, Wq[row0:row0 + rows], sw[row0:row0 + rows]))
    lin = sharded.NShardedLinear(N, K, rank, world, w.shard_rows, compute)
    Y = lin(torch.from_numpy(X))
    xq, xs, _ = O.quantize_x_q8(X)
    full = O.gemm_mmq_w4a8(xq, xs, Wq, sw)
    assert Y.shape == (M, N) and np.array_equal(Y.numpy().view(np.uint32), full.view(np.uint32)), (M, N, K, rank)
# expert shards: each rank computes the down outputs of the slots routed to its experts, the rows are exchanged, every
# rank combines in the fixed order; equal, bit for bit, to the whole block on one rank
S, topk, E, H, MI = 6, 2, 4, 64, 32
rng = np.random.default_rng(11)
n2 = O.make_activations(S, H, seed=3)
gu_wq, gu_sc = O.make_weights(E * 2 * MI, H, seed=4); dn_wq, dn_sc = O.make_weights(E * H, MI, seed=5)
gu_wq, gu_sc = gu_wq.reshape(E, 2 * MI, -1), (gu_sc * 8).reshape(E, 2 * MI, -1)
dn_wq, dn_sc = dn_wq.reshape(E, H, -1), dn_sc.reshape(E, H, -1)
idx = np.stack([rng.permutation(E)[:topk] for _ in range(S)]).astype(np.int32).reshape(-1)
dw = rng.random(S * topk).astype(np.float32)
whole = O.moe_block_w4a8(n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw, topk)
def compute(n2t, idxt, base, count):
    so = whole["so"].copy()                                   # a slot's row depends only on its own expert ...
    mine = (idxt.numpy() >= base) & (idxt.numpy() < base + count)
    so[~mine] = 0.0                                           # ... and a rank produces only its experts' slots
    return torch.from_numpy(so)
blk = sharded.ExpertShardedBlock(E, topk, rank, world, compute)
out = blk(torch.from_numpy(n2), torch.from_numpy(idx), torch.from_numpy(dw))
assert np.array_equal(out.numpy().view(np.uint32), whole["out"].view(np.uint32)), rank
assert sharded.expert_range(E, rank, world) == (rank * (E // world), E // world)
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_n_sharded_all_gather_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text("ROOT = %r\n" % ROOT + _WORKER)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29611", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=240)[0] for p in procs]
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o[-2000:]
        assert "rank %d ok" % r in o


_SHIM_TU = r'''
#include "kernels/quantize_x.cuh"
#include "kernels/gemv_w4a8.cuh"
#include "kernels/gemm_batch.cuh"
#include "kernels/gemm_mma.cuh"
#include "kernels/gemm_mmq.cuh"
#include "kernels/gemm_mmq_tmpl.cuh"
#include "kernels/gemm_mmq_raster.cuh"
#include "kernels/gemm_mmq_ms.cuh"
#include "kernels/moe_w4a8.cuh"
#include "runtime/weights_shard.h"
__global__ void helpers(int *o) { o[0] = w4a8_pk(0x21, 0x43); o[1] = mmq_unpack4v(0x4321u); }   // device helpers other reference files borrow
// every launcher of the reference's W4A8 path, called with the reference's argument lists and defaults
void all(const float *X, int8_t *xq, float *xs, int32_t *xsum, const uint8_t *Wq, const void *sw, float *Y, cudaStream_t st) {
    launch_quantize_x_q8(X, xq, xs, xsum, 64, 1);
    launch_gemv_w4a8(xq, xs, xsum, Wq, sw, Y, 64, 8, 1);
    launch_gemv_w4a8_mlp<2>(xq, xs, xsum, Wq, sw, Y, 64, 8, 1, 0, st);
    launch_gemv_w4a8_mlp_auto(xq, xs, xsum, Wq, sw, Y, 64, 8, 1, 1, st);
    launch_gemv_w4a8_g4(xq, xs, xsum, Wq, sw, Y, 64, 8, 1, 0, st);
    launch_gemv_w4a8_sb(xq, xs, Wq, sw, Y, 64, 8, 5);
    launch_gemv_w4a8_sb_g4(xq, xs, Wq, sw, Y, 64, 8, 5, 0, st);
    launch_gemm_batch_w4a8(xq, xs, Wq, sw, Y, 64, 8, 16);
    launch_gemm_mma_w4a8(xq, xs, Wq, sw, Y, 128, 8, 64);
    launch_gemm_mma_w4a8_bm<128>(xq, xs, Wq, sw, Y, 128, 8, 64, 0, st);
    launch_gemm_mmq_w4a8(xq, xs, Wq, sw, Y, 128, 8, 64);
    launch_gemm_mmq_w4a8_kt<128>(xq, xs, Wq, sw, Y, 128, 8, 64, 0, st);
    launch_gemm_mmq_w4a8_auto(xq, xs, Wq, sw, Y, 128, 8, 64);
    launch_gemm_mmq_tmpl<256, 64, 64, 4, 2>(xq, xs, Wq, sw, Y, 128, 8, 64, 0, st);
    launch_gemm_mmq_raster_w4a8(xq, xs, Wq, sw, Y, 128, 8, 64, 0, 1, 1);
    launch_gemm_mmq_ms<128, 128, 64, 2, 4, 3>(xq, xs, Wq, sw, Y, 128, 8, 64);
    launch_gemm_bm16_splitk(xq, xs, Wq, sw, Y, 16, 8, 64);
    // the W4A8 form of the fused routed-expert path at models/moe_block.cuh:45-52 (tensor names as there)
    launch_moe_w4a8_block(X, Wq, sw, Wq, sw, (const int *)xsum, X, Y, /*S=*/4, /*H=*/64, /*MI=*/32, /*E=*/8, /*K=*/2, 0);
    QMatShard m = mat_shard("dir", "L0_mlp.gate_proj", 8, 64, 0, 0, 1);
    (void)m;
}
int main() { return QBLK == 32 ? 0 : 1; }
'''


def test_shim_headers_compile_and_link_with_reference_signatures(w4a8, tmp_path):
    nvcc = "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not available")
    src = tmp_path / "shim_tu.cu"
    src.write_text(_SHIM_TU)
    pkg = os.path.join(ROOT, "dgx-serving_b200")
    exe = tmp_path / "shim_tu"
    r = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-I" + pkg, "-o", str(exe), str(src),
                        "-L" + pkg, "-lw4a8_b200", "-Xlinker", "-rpath", "-Xlinker", pkg], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
    assert subprocess.run([str(exe)]).returncode == 0
