"""Routed-expert block in W4A8 (w4a8_moe_block / w4a8_moe_block_shard) against the CPU oracle, stage by stage.

The block replaces the reference's four fused launches (models/moe_block.cuh:45-52, kernels/moe_fused.cuh:14-76) with the
expert products in W4A8.  What is bit-exact: the sort (a stable counting sort), the gate|up and down products of the
sorted grouped GEMM against oracle_moe_w4a8 (MMQ order per slot), the quantization of the block's own fp32 hidden
activations, and the fixed-order combine.  The grouped GEMV used for few slots has the single-row GEMV's own fp32 order
(bit-exact against that order per slot, within the 1e-5 gate against MMQ order).  The activation itself uses the GPU's
expf, which may differ from the C library's by an ulp, so the hidden activations are compared within a tolerance and
the stages after them are checked on the block's own intermediates.
"""
import numpy as np
import pytest
import torch

from conftest import to_dev
from test_gpu_parity import REL_TOL, rel_err

pytestmark = pytest.mark.gpu


def make_block(oracle, S, topk, E, H, MI, seed, sd=0):
    rng = np.random.default_rng(seed)
    n2 = oracle.make_activations(S, H, seed=seed + 1, outliers=True)
    gu_wq, gu_sc = oracle.make_weights(E * 2 * MI, H, seed=seed + 2, scale_dtype=sd)
    dn_wq, dn_sc = oracle.make_weights(E * H, MI, seed=seed + 3, scale_dtype=sd)
    gu_sc = (gu_sc.astype(np.float32) * 8.0).astype(gu_sc.dtype)   # gate/up outputs of order 1, so the activation is exercised
    idx = np.stack([rng.permutation(E)[:topk] for _ in range(S)]).astype(np.int32).reshape(-1)
    dw = rng.random(S * topk).astype(np.float32)
    dw /= dw.reshape(S, topk).sum(axis=1).repeat(topk)
    return n2, gu_wq.reshape(E, 2 * MI, H // 2), gu_sc.reshape(E, 2 * MI, H // 32), dn_wq.reshape(E, H, MI // 2), dn_sc.reshape(E, H, MI // 32), idx, dw


def ws_view(ws, off, shape, dtype):
    n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
    return ws[off:off + n].view(dtype).reshape(shape)


def run_block(w4a8, cuda, case, S, topk, E, H, MI, kernel, sd=0, act=0):
    n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw = case
    lay = w4a8.moe_layout_for(S, topk, H, MI, E)
    ws = torch.full((lay.bytes,), 0x7F, dtype=torch.uint8, device=cuda)
    out = torch.full((S, H), float("nan"), dtype=torch.float32, device=cuda)
    d = [to_dev(a, cuda) for a in (n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw)]
    w4a8.config("moe_kernel", kernel)
    try:
        w4a8.moe_block(d[0], d[1], d[2], d[3], d[4], d[5], d[6], out, S, topk, H, MI, E, ws, sd, act)
        torch.cuda.synchronize()
        w4a8.device_status()
    finally:
        w4a8.config("moe_kernel", 0)
    return lay, ws, out


def check_stages(oracle, case, lay, ws, out, S, topk, E, H, MI, gemm, act=0):
    n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw = case
    nslots = S * topk
    ref = oracle.moe_block_w4a8(n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw, topk, act)
    xq = ws_view(ws, lay.xq, (S, H), torch.int8).cpu().numpy()
    xs = ws_view(ws, lay.xs, (S, H // 32), torch.float32).cpu().numpy()
    assert np.array_equal(xq, ref["xq"]) and np.array_equal(xs.view(np.uint32), ref["xs"].view(np.uint32))
    if gemm:
        perm = ws_view(ws, lay.perm, (nslots,), torch.int32).cpu().numpy()
        pos = ws_view(ws, lay.pos, (nslots,), torch.int32).cpu().numpy()
        offs = ws_view(ws, lay.offsets, (E + 1,), torch.int32).cpu().numpy()
        order = np.argsort(idx, kind="stable")                       # the stable sort by expert
        assert np.array_equal(perm, order) and np.array_equal(pos[perm], np.arange(nslots))
        assert np.array_equal(offs, np.concatenate([[0], np.cumsum(np.bincount(idx, minlength=E))]))
        n_items = int(ws_view(ws, lay.num_items, (1,), torch.int32).item())
        items = ws_view(ws, lay.items, (n_items, 4), torch.int32).cpu().numpy()
        assert n_items == int(np.sum((np.bincount(idx, minlength=E) + 63) // 64))        # an expert's rows in tiles of up to 64
        assert np.all(items[:, 2] >= 1) and np.all(items[:, 2] <= 64) and int(items[:, 2].sum()) == nslots
    else:
        pos = np.arange(nslots)
    gu = ws_view(ws, lay.gu, (nslots, 2 * MI), torch.float32).cpu().numpy()[pos]
    if gemm:
        assert np.array_equal(gu.view(np.uint32), ref["gu"].view(np.uint32))
    else:
        assert rel_err(gu, ref["gu"]) < REL_TOL
        for slot in (0, nslots // 2, nslots - 1):
            e, tok = idx[slot], slot // topk
            r = oracle.gemv_b200_order(ref["xq"][tok:tok + 1], ref["xs"][tok:tok + 1], gu_wq[e].reshape(2 * MI, -1), gu_sc[e].reshape(2 * MI, -1))
            assert np.array_equal(gu[slot].view(np.uint32), r[0].view(np.uint32))
    # hidden activations: act(gate) * up of the block's own gate|up outputs, then quantized
    hid = oracle.glu(gu[:, :MI], gu[:, MI:], act)
    xq_h = ws_view(ws, lay.xq_h, (nslots, MI), torch.int8).cpu().numpy()[pos]
    xs_h = ws_view(ws, lay.xs_h, (nslots, MI // 32), torch.float32).cpu().numpy()[pos]
    xq_o, xs_o, _ = oracle.quantize_x_q8(hid)
    assert np.allclose(xs_h, xs_o, rtol=1e-5, atol=0)
    diff = np.abs(xq_h.astype(np.int32) - xq_o.astype(np.int32))
    assert diff.max() <= 1 and np.mean(diff != 0) < 2e-3
    # down product on the block's own quantized hidden activations
    so = ws_view(ws, lay.sout, (nslots, H), torch.float32).cpu().numpy()[pos]
    so_ref = oracle.moe_w4a8(xq_h, xs_h, dn_wq.reshape(E * H, -1), dn_sc.reshape(E * H, -1), idx, topk, 1, H, MI)
    if gemm:
        assert np.array_equal(so.view(np.uint32), so_ref.view(np.uint32))
    else:
        assert rel_err(so, so_ref) < REL_TOL
        slot = nslots - 1
        e = idx[slot]
        r = oracle.gemv_b200_order(xq_h[slot:slot + 1], xs_h[slot:slot + 1], dn_wq[e].reshape(H, -1), dn_sc[e].reshape(H, -1))
        assert np.array_equal(so[slot].view(np.uint32), r[0].view(np.uint32))
    # router weight + combine in ascending k: bit-exact on the block's own down outputs
    y = out.cpu().numpy()
    assert np.array_equal(y.view(np.uint32), oracle.moe_combine(so, dw, topk).view(np.uint32))
    # and the whole block against the oracle's: differences come only from the activation's last bit flipping a
    # quantized hidden value here and there
    assert rel_err(y, ref["out"]) < 2e-3
    return ref


@pytest.mark.parametrize("S,topk,E,H,MI,kernel,sd", [
    (8, 8, 128, 2048, 768, 1, 0),       # benchmark configuration 5 (128 experts, top-8) at M = 8: grouped GEMV
    (8, 8, 128, 2048, 768, 2, 0),       # the same through the sorted grouped GEMM
    (37, 3, 5, 256, 96, 2, 0),          # ragged: partial tiles, MI not a multiple of the K-tile
    (37, 3, 5, 256, 96, 1, 1),          # fp16 scales, GEMV path
    (300, 3, 3, 128, 64, 2, 1),         # every expert gets 300 rows: five tiles per expert, fp16 scales
    (5, 2, 7, 160, 32, 0, 0),           # auto
    (5, 2, 7, 256, 768, 1, 1),          # MI = 768 on the GEMV path: both activation rows produced inside the GEMVs (H <= 1024), fp16 scales
    (3, 4, 6, 1536, 768, 0, 0),         # the same with two groups per lane in gate|up
    (40, 2, 300, 64, 32, 2, 0),         # more experts than the sort kernel's per-warp histograms hold
])
def test_moe_block_stages(w4a8, oracle, cuda, S, topk, E, H, MI, kernel, sd):
    case = make_block(oracle, S, topk, E, H, MI, seed=300 + S + E, sd=sd)
    lay, ws, out = run_block(w4a8, cuda, case, S, topk, E, H, MI, kernel, sd)
    gemm = kernel == 2 or (kernel == 0 and S * topk > 128)
    check_stages(oracle, case, lay, ws, out, S, topk, E, H, MI, gemm)


def test_moe_block_config5_m512(w4a8, oracle, cuda):
    """benchmark configuration 5 (128 experts, top-8) at M = 512: 128 experts, top-8, H = 2048, MI = 768 — 4096 slots through the sorted grouped GEMM,
    every stage against the oracle."""
    S, topk, E, H, MI = 512, 8, 128, 2048, 768
    case = make_block(oracle, S, topk, E, H, MI, seed=512)
    lay, ws, out = run_block(w4a8, cuda, case, S, topk, E, H, MI, 0)
    check_stages(oracle, case, lay, ws, out, S, topk, E, H, MI, True)
    # a second call on the same workspace gives the same bits (nothing accumulates across calls)
    lay2, ws2, out2 = run_block(w4a8, cuda, case, S, topk, E, H, MI, 2)
    assert torch.equal(out.view(torch.int32), out2.view(torch.int32))


def test_moe_block_geglu_and_unused_experts(w4a8, oracle, cuda):
    """act = 1 (GeGLU, the Gemma expert activation) and a routing that leaves most experts without a slot."""
    S, topk, E, H, MI = 40, 2, 64, 128, 64
    case = list(make_block(oracle, S, topk, E, H, MI, seed=77))
    rng = np.random.default_rng(5)
    case[5] = np.stack([rng.permutation(6)[:topk] * 9 for _ in range(S)]).astype(np.int32).reshape(-1)   # experts 0, 9, ..., 45 only
    lay, ws, out = run_block(w4a8, cuda, case, S, topk, E, H, MI, 2, act=1)
    check_stages(oracle, case, lay, ws, out, S, topk, E, H, MI, True, act=1)


def test_moe_block_geglu_inside_the_down_gemv(w4a8, oracle, cuda):
    """act = 1 on the decode path whose down GEMV computes the activation in its prologue (MI = 768, H <= 2048)."""
    S, topk, E, H, MI = 6, 2, 8, 512, 768
    case = make_block(oracle, S, topk, E, H, MI, seed=78)
    lay, ws, out = run_block(w4a8, cuda, case, S, topk, E, H, MI, 1, act=1)
    check_stages(oracle, case, lay, ws, out, S, topk, E, H, MI, False, act=1)


def test_moe_gemv_idx_written_on_the_stream(w4a8, oracle, cuda):
    """The routing indices may be produced by a kernel enqueued on the same stream right before the grouped GEMV (the
    router / top-k of models/moe_block.cuh:40-41): the GEMV's CTAs start early under programmatic dependent launch but
    read idx only after the stream dependency is resolved."""
    tokens, topk, E, N, K = 8, 8, 128, 768, 2048
    rng = np.random.default_rng(3)
    idx = np.stack([rng.permutation(E)[:topk] for _ in range(tokens)]).astype(np.int32).reshape(-1)
    nslots = tokens * topk
    X = oracle.make_activations(tokens, K, seed=5)
    Wq, sw = oracle.make_weights(E * N, K, seed=6)
    xq, xs, _ = oracle.quantize_x_q8(X)
    d = [to_dev(a, cuda) for a in (xq, xs, Wq, sw)]
    src = to_dev(idx, cuda)
    big = torch.zeros(64 << 20, dtype=torch.float32, device=cuda)
    ref = oracle.moe_w4a8(xq, xs, Wq, sw, idx, topk, 0, N, K)
    for rep in range(5):
        idx_d = torch.full((nslots,), E + 5, dtype=torch.int32, device=cuda)      # invalid ids: a too-early read leaves Y untouched
        Y = torch.full((nslots, N), float("nan"), dtype=torch.float32, device=cuda)
        torch.cuda.synchronize()
        big.add_(1.0)                                                                # keeps the stream busy for a while
        torch.add(src, 0, out=idx_d)                                                 # a kernel writes idx ...
        w4a8.moe_gemv(d[0], d[1], d[2], d[3], idx_d, Y, nslots, topk, 0, N, K, E)    # ... right before the GEMV reads it
        torch.cuda.synchronize()
        assert rel_err(Y.cpu().numpy(), ref) < REL_TOL


def test_moe_block_argument_checks(w4a8, cuda):
    lay = w4a8.moe_layout_for(4, 2, 64, 32, 4)
    ws = torch.empty(lay.bytes, dtype=torch.uint8, device=cuda)
    f = torch.zeros(4 * 64, dtype=torch.float32, device=cuda)
    b = torch.zeros(1 << 16, dtype=torch.uint8, device=cuda)
    i = torch.zeros(8, dtype=torch.int32, device=cuda)
    with pytest.raises(w4a8.W4A8Error):
        w4a8.moe_block(f, b, f, b, f, i, f, f, 4, 2, 48, 32, 4, ws)              # H not a multiple of 32
    with pytest.raises(w4a8.W4A8Error):
        w4a8.moe_block(f, b, f, b, f, i, f, f, 4, 2, 64, 32, 4, ws[:1024])       # workspace too small
    with pytest.raises(w4a8.W4A8Error):
        w4a8.moe_block(f, b, f, b, f, None, f, f, 4, 2, 64, 32, 4, ws)           # no routing indices
    with pytest.raises(w4a8.W4A8Error):
        w4a8.moe_layout_for(4, 2, 64, 32, 5000)                                   # more experts than the sort kernel takes
    w4a8.moe_block(f, b, f, b, f, i, f, f, 0, 2, 64, 32, 4, ws)                  # no tokens: nothing to do
    with pytest.raises(w4a8.W4A8Error):
        w4a8.config("moe_kernel", 3)


def test_moe_block_expert_shard_emulated(w4a8, oracle, cuda):
    """Eight expert shards driven one after the other on one GPU (phase 1 on every rank, then phase 2 on every rank):
    every rank ends with the whole block output, bit-identical to the single-GPU block with all experts."""
    S, topk, E, H, MI, world = 24, 4, 32, 256, 96, 8
    case = make_block(oracle, S, topk, E, H, MI, seed=88)
    n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw = case
    for kernel in (1, 2):
        lay1, ws1, out1 = run_block(w4a8, cuda, case, S, topk, E, H, MI, kernel)
        nslots, per = S * topk, E // world
        sbytes = nslots * H * 4
        arenas = [w4a8.Arena(sbytes, r, world) for r in range(world)]
        try:
            for a in arenas:
                a.connect_pointers([b.base for b in arenas])
                a.tensor(0, (nslots, H)).fill_(float("nan"))
            lay = w4a8.moe_layout_for(S, topk, H, MI, per)
            wss = [torch.empty(lay.bytes, dtype=torch.uint8, device=cuda) for _ in range(world)]
            outs = [torch.full((S, H), float("nan"), dtype=torch.float32, device=cuda) for _ in range(world)]
            shared = [to_dev(a, cuda) for a in (n2, idx, dw)]
            shards = [[to_dev(np.ascontiguousarray(t[r * per:(r + 1) * per]), cuda) for t in (gu_wq, gu_sc, dn_wq, dn_sc)] for r in range(world)]
            w4a8.config("moe_kernel", kernel)
            for phase in (1, 2):
                for r in range(world):
                    g = shards[r]
                    w4a8.moe_block_shard(shared[0], g[0], g[1], g[2], g[3], shared[1], shared[2], outs[r], S, topk, H, MI, r * per, per,
                                         wss[r], arenas[r], 0, 1, timeout_us=2000000, phase=phase)
            torch.cuda.synchronize()
            w4a8.device_status()
            for r in range(world):
                assert torch.equal(outs[r].view(torch.int32), out1.view(torch.int32)), (kernel, r)
        finally:
            w4a8.config("moe_kernel", 0)
            for a in arenas:
                a.close()


_SHARD_WORKER = r'''
import os, sys
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, os.path.join(ROOT, "oracle"))
import numpy as np, torch, torch.distributed as dist
from conftest import load_package, to_dev
from test_gpu_moe import make_block
import oracle as O
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
w = load_package()
epoch = 0
for (S, topk, E, H, MI) in [(8, 8, 128, 2048, 768), (96, 4, 16, 256, 96)]:      # grouped GEMV, then the sorted grouped GEMM
    case = make_block(O, S, topk, E, H, MI, seed=900 + S)
    n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw = case
    nslots, per = S * topk, E // world
    d = [to_dev(a, dev) for a in (n2, gu_wq, gu_sc, dn_wq, dn_sc, idx, dw)]
    lay1 = w.moe_layout_for(S, topk, H, MI, E)
    ws1 = torch.empty(lay1.bytes, dtype=torch.uint8, device=dev)
    out1 = torch.empty((S, H), dtype=torch.float32, device=dev)
    w.moe_block(d[0], d[1], d[2], d[3], d[4], d[5], d[6], out1, S, topk, H, MI, E, ws1)     # all experts on this GPU
    sbytes = (nslots * H * 4 + 255) // 256 * 256
    a = w.Arena(2 * sbytes, rank, world)
    handles = [None] * world
    dist.all_gather_object(handles, a.export_handle())
    a.connect_handles(handles)
    dist.barrier()
    lay = w.moe_layout_for(S, topk, H, MI, per)
    ws = torch.empty(lay.bytes, dtype=torch.uint8, device=dev)
    sh = [to_dev(np.ascontiguousarray(t[rank * per:(rank + 1) * per]), dev) for t in (gu_wq, gu_sc, dn_wq, dn_sc)]
    for step in range(4):
        epoch += 1
        out = torch.full((S, H), float("nan"), dtype=torch.float32, device=dev)
        a.tensor((step % 2) * sbytes, (nslots, H)).fill_(float("nan"))
        torch.cuda.synchronize(); dist.barrier()
        w.moe_block_shard(d[0], sh[0], sh[1], sh[2], sh[3], d[5], d[6], out, S, topk, H, MI, rank * per, per, ws, a,
                          (step % 2) * sbytes, step + 1, timeout_us=2000000)
        torch.cuda.synchronize()
        w.device_status()
        assert torch.equal(out.view(torch.int32), out1.view(torch.int32)), (S, step, rank)
        dist.barrier()
    a.close()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


@pytest.mark.parametrize("world", [2, 8])
def test_moe_block_expert_shard_real_gpus(tmp_path, world):
    """Real ranks, one process per GPU (skipped when the box has fewer GPUs): 128 experts split over the ranks, the
    slots' down outputs exchanged through the arenas, every rank's block output bit-identical to the single-GPU block."""
    import os
    import subprocess
    import sys
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "worker.py"
    script.write_text("ROOT = %r\n" % root + _SHARD_WORKER)
    procs = []
    try:
        for r in range(world):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                       MASTER_PORT=str(29833 + world), NCCL_NVLS_ENABLE="0")
            procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        outs = [p.communicate(timeout=600)[0] for p in procs]
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
                p.wait()
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o[-3000:]
        assert "rank %d ok" % r in o
