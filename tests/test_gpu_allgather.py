"""GPU tests of the N-sharded GEMV with the all-gather fused into the epilogue (w4a8_gemv_allgather).

One GPU: the two ranks are emulated in one process, one after the other on one stream — each "rank" owns an arena,
both arenas are mapped into each other by plain pointers, rank 0's kernel runs, then rank 1's, then both waits — so no
kernel ever waits for a kernel that is not already complete.  The bounded wait is exercised with a flag nothing sets:
it must give up, report W4A8_ERR_DEVICE and leave the context usable.  Two, four or eight GPUs (skipped on a smaller box): real ranks
as child processes with CUDA IPC mappings, NVLS off, checked against the oracle and against the NCCL all-gather path.
"""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import to_dev
from test_gpu_parity import gemv_expected, make_case

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("S,N,K", [(1, 520, 512), (5, 520, 512), (16, 1000, 1024), (20, 264, 256), (3, 37, 96), (1, 1000, 2048)])
def test_fused_allgather_ranks_emulated(w4a8, oracle, cuda, S, N, K, world):
    """`world` ranks emulated on one GPU: their kernels run one after the other over `world` arenas (never two waiting
    kernels at once), then every rank's wait finds all flags set."""
    xq, xs, Wq, sw = make_case(oracle, S, N, K, seed=31 + S + N)
    xq_d, xs_d = to_dev(xq, cuda), to_dev(xs, cuda)
    ybytes = S * N * 4
    ystride = (ybytes + 255) // 256 * 256
    arenas = [w4a8.Arena(2 * ystride, r, world) for r in range(world)]
    try:
        for a in arenas:
            a.connect_pointers([b.base for b in arenas])
        shards = []
        for r in range(world):
            row0, rows = w4a8.shard_rows(N, r, world)
            shards.append((row0, rows, to_dev(Wq[row0:row0 + rows], cuda), to_dev(sw[row0:row0 + rows], cuda)))
        expect = gemv_expected(oracle, xq, xs, Wq, sw)
        for epoch in (1, 2, 3):                                   # alternate the two Y buffers, reuse included
            off = (epoch % 2) * ystride
            for r, a in enumerate(arenas):
                row0, rows, Wq_r, sw_r = shards[r]
                a.gemv_allgather(xq_d, xs_d, Wq_r, sw_r, off, K, rows, row0, N, S, 0, epoch)
            for a in arenas:
                a.wait(epoch, timeout_us=200000)
            w4a8.device_status()
            for a in arenas:                                      # every rank holds the complete Y
                y = a.tensor(off, (S, N)).cpu().numpy()
                assert np.array_equal(y.view(np.uint32), expect.view(np.uint32))
                a.tensor(off, (S, N)).fill_(float("nan"))
    finally:
        for a in arenas:
            a.close()


@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("M,N,K,scale_dtype", [(130, 520, 512, 0), (17, 264, 256, 1), (300, 1000, 1024, 0), (64, 37 * 4, 96, 0)])
def test_fused_gemm_allgather_ranks_emulated(w4a8, oracle, cuda, M, N, K, scale_dtype, world):
    """The GEMM with the peer-store epilogue: `world` ranks emulated on one GPU, kernels one after the other; every
    rank's arena ends up with the whole Y[M, N], bit-identical to w4a8_gemm on the unsharded matrix (MMQ order)."""
    xq, xs, Wq, sw = make_case(oracle, M, N, K, seed=77 + M + N, scale_dtype=scale_dtype)
    xq_d, xs_d = to_dev(xq, cuda), to_dev(xs, cuda)
    ystride = (M * N * 4 + 255) // 256 * 256
    arenas = [w4a8.Arena(2 * ystride, r, world) for r in range(world)]
    try:
        for a in arenas:
            a.connect_pointers([b.base for b in arenas])
        shards = []
        for r in range(world):
            row0, rows = w4a8.shard_rows(N, r, world)
            shards.append((row0, rows, to_dev(Wq[row0:row0 + rows], cuda), to_dev(sw[row0:row0 + rows], cuda)))
        expect = oracle.gemm_mmq_w4a8(xq, xs, Wq, sw)
        for epoch in (1, 2):
            off = (epoch % 2) * ystride
            for r, a in enumerate(arenas):
                row0, rows, Wq_r, sw_r = shards[r]
                a.gemm_allgather(xq_d, xs_d, Wq_r, sw_r, off, M, rows, row0, N, K, scale_dtype, epoch)
            for a in arenas:
                a.wait(epoch, timeout_us=200000)
            w4a8.device_status()
            for a in arenas:
                y = a.tensor(off, (M, N)).cpu().numpy()
                assert np.array_equal(y.view(np.uint32), expect.view(np.uint32))
                a.tensor(off, (M, N)).fill_(float("nan"))
    finally:
        for a in arenas:
            a.close()


def test_allgather_wait_gives_up_and_reports(w4a8, oracle, cuda):
    """Failure detection without a GPU fault: a flag that nothing sets makes the bounded wait run out."""
    arenas = [w4a8.Arena(4096, r, 2) for r in range(2)]
    try:
        for a in arenas:
            a.connect_pointers([b.base for b in arenas])
        arenas[0].wait(7, timeout_us=2000)                        # nobody published epoch 7
        with pytest.raises(w4a8.W4A8Error) as ei:
            w4a8.device_status()
        assert ei.value.code == w4a8.ERR_DEVICE and "0x20" in str(ei.value)
        w4a8.device_status()                                      # the error word was cleared; the context still works
        xq, xs, Wq, sw = make_case(oracle, 2, 64, 256, seed=3)
        Y = torch.empty((2, 64), dtype=torch.float32, device=cuda)
        w4a8.launch_gemv_w4a8_sb(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq, cuda), to_dev(sw, cuda), Y, 256, 64, 2)
        torch.cuda.synchronize()
        assert np.array_equal(Y.cpu().numpy().view(np.uint32), gemv_expected(oracle, xq, xs, Wq, sw).view(np.uint32))
    finally:
        for a in arenas:
            a.close()


def test_in_kernel_wait_gives_up_and_reports(w4a8, oracle, cuda):
    """The wait folded into the GEMV (w4a8_gemv_allgather_sync) is bounded too: rank 1 of the emulated pair never runs, so
    rank 0's threads poll 2 ms for slots nothing fills, record the error and return; the outputs rank 0 computed are in
    place, rank 1's part of Y is untouched, the context stays usable."""
    S, N, K = 1, 520, 512
    xq, xs, Wq, sw = make_case(oracle, S, N, K, seed=11)
    arenas = [w4a8.Arena(8192, r, 2) for r in range(2)]
    try:
        for a in arenas:
            a.connect_pointers([b.base for b in arenas])
        row0, rows = w4a8.shard_rows(N, 0, 2)
        arenas[0].tensor(0, (S, N)).fill_(float("nan"))
        arenas[0].gemv_allgather_sync(to_dev(xq, cuda), to_dev(xs, cuda), to_dev(Wq[row0:row0 + rows], cuda), to_dev(sw[row0:row0 + rows], cuda),
                                      0, K, rows, row0, N, S, 0, 1, 2000)
        with pytest.raises(w4a8.W4A8Error) as ei:
            w4a8.device_status()
        assert ei.value.code == w4a8.ERR_DEVICE and "0x20" in str(ei.value)
        w4a8.device_status()                                      # cleared; the context still works
        expect = gemv_expected(oracle, xq, xs, Wq, sw)
        y = arenas[0].tensor(0, (S, N)).cpu().numpy()
        assert np.array_equal(y[:, row0:row0 + rows].view(np.uint32), expect[:, row0:row0 + rows].view(np.uint32))
        assert np.all(np.isnan(y[:, row0 + rows:])) and np.all(np.isnan(y[:, :row0]))
    finally:
        for a in arenas:
            a.close()


_WORKER = r'''
import os, sys
sys.path.insert(0, os.path.join(ROOT, "tests")); sys.path.insert(0, os.path.join(ROOT, "oracle"))
import numpy as np, torch, torch.distributed as dist
from conftest import load_package, to_dev
from test_gpu_parity import gemv_expected, make_case
import importlib
import oracle as O
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
w = load_package()
sharded = importlib.import_module("dgx_serving_b200.sharded")
for (S, N, K) in [(1, 17408, 5120), (8, 4096, 1024), (16, 1001, 512), (1, 1, 256), (2, 3, 256)]:   # the last two leave ranks without rows
    xq, xs, Wq, sw = make_case(O, S, N, K, seed=5 + S)
    expect = gemv_expected(O, xq, xs, Wq, sw)
    row0, rows = w.shard_rows(N, rank, world)
    xq_d, xs_d = to_dev(xq, dev), to_dev(xs, dev)
    Wq_r, sw_r = to_dev(Wq[row0:row0 + rows], dev), to_dev(sw[row0:row0 + rows], dev)
    ystride = (S * N * 4 + 255) // 256 * 256
    a = w.Arena(2 * ystride, rank, world)
    handles = [None] * world
    dist.all_gather_object(handles, a.export_handle())
    a.connect_handles(handles)
    dist.barrier()
    for epoch in range(1, 9):
        off = (epoch % 2) * ystride
        if epoch <= 4:                                     # exchange and a wait kernel of its own
            a.gemv_allgather(xq_d, xs_d, Wq_r, sw_r, off, K, rows, row0, N, S, 0, epoch)
            a.wait(epoch, timeout_us=2000000)
        else:                                              # the wait folded into the call's last kernel
            a.gemv_allgather_sync(xq_d, xs_d, Wq_r, sw_r, off, K, rows, row0, N, S, 0, epoch, 2000000)
        w.device_status()
        y = a.tensor(off, (S, N)).cpu().numpy()
        assert np.array_equal(y.view(np.uint32), expect.view(np.uint32)), (S, N, K, epoch, rank)
        a.tensor(off, (S, N)).fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()                                     # nobody refills a buffer a peer is still checking
    # the NCCL path gives the same bits
    Yloc = torch.empty((S, rows), dtype=torch.float32, device=dev)
    w.launch_gemv_w4a8_sb(xq_d, xs_d, Wq_r, sw_r, Yloc, K, rows, S)
    Y = sharded.all_gather_columns(Yloc, sharded.shard_plan(N, world, w.shard_rows))
    assert np.array_equal(Y.cpu().numpy().view(np.uint32), expect.view(np.uint32))
    dist.barrier()
    a.close()
# the prefill GEMM with the fused exchange: every rank ends up with the whole Y[M, N] in MMQ order
for (M, N, K) in [(256, 1024, 1024), (130, 520, 512)]:
    xq, xs, Wq, sw = make_case(O, M, N, K, seed=9 + M)
    expect = O.gemm_mmq_w4a8(xq, xs, Wq, sw)
    row0, rows = w.shard_rows(N, rank, world)
    xq_d, xs_d = to_dev(xq, dev), to_dev(xs, dev)
    Wq_r, sw_r = to_dev(Wq[row0:row0 + rows], dev), to_dev(sw[row0:row0 + rows], dev)
    ystride = (M * N * 4 + 255) // 256 * 256
    a = w.Arena(2 * ystride, rank, world)
    handles = [None] * world
    dist.all_gather_object(handles, a.export_handle())
    a.connect_handles(handles)
    dist.barrier()
    for epoch in range(1, 6):
        off = (epoch % 2) * ystride
        if epoch <= 3:
            a.gemm_allgather(xq_d, xs_d, Wq_r, sw_r, off, M, rows, row0, N, K, 0, epoch)
            a.wait(epoch, timeout_us=2000000)
        else:
            a.gemm_allgather_sync(xq_d, xs_d, Wq_r, sw_r, off, M, rows, row0, N, K, 0, epoch, 2000000)
        w.device_status()
        y = a.tensor(off, (M, N)).cpu().numpy()
        assert np.array_equal(y.view(np.uint32), expect.view(np.uint32)), (M, N, K, epoch, rank)
        a.tensor(off, (M, N)).fill_(float("nan"))
        torch.cuda.synchronize()
        dist.barrier()
    dist.barrier()
    a.close()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_allgather_real_gpus(tmp_path, world):
    """Real ranks, one process per GPU (skipped when the box has fewer GPUs than `world`)."""
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    script = tmp_path / "worker.py"
    script.write_text("ROOT = %r\n" % ROOT + _WORKER)
    procs = []
    try:
        for r in range(world):
            env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                       MASTER_PORT=str(29733 + world), NCCL_NVLS_ENABLE="0")
            procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
        outs = [p.communicate(timeout=600)[0] for p in procs]
    finally:
        for p in procs:                                    # never leave a rank behind in a barrier, holding a GPU
            if p.poll() is None:
                p.kill()
                p.wait()
    for r, (p, o) in enumerate(zip(procs, outs)):
        assert p.returncode == 0, o[-3000:]
        assert "rank %d ok" % r in o
