"""N-sharded (column tensor-parallel) W4A8 linear: host-side plumbing over torch.distributed.

Every output column n of Y = X * W^T depends only on row n of Wq / sw, and rows are the outer dimension of
the reference's weight files (runtime/weights_qwen.cu:28-36), so rank r of g keeps the contiguous row range
w4a8_shard_rows gives it, computes Y[:, row0:row0+rows] with the ordinary single-GPU entry points and one
all-gather reassembles the row-major Y[M, N].  The reference itself is single-GPU; nothing here replaces
reference code.  The collective is NCCL on GPUs (gloo in the CPU tests); there is no other data-path exchange.
"""
import torch
import torch.distributed as dist


def shard_plan(N, world, shard_rows):
    """[(row0, rows)] for every rank, from the library's w4a8_shard_rows (passed in as `shard_rows`)."""
    plan = [shard_rows(N, r, world) for r in range(world)]
    assert plan[0][0] == 0 and sum(r for _, r in plan) == N
    for (a0, a), (b0, _) in zip(plan, plan[1:]):
        assert a0 + a == b0, "shards must be contiguous and ordered by rank"
    return plan


def all_gather_columns(Y_local, plan, group=None):
    """Y_local[M, rows_r] on every rank -> Y[M, N] on every rank (row-major).

    Equal shards use one all_gather_into_tensor into [g][M][rows] followed, for M > 1, by the permutation to
    [M][g*rows]; for M = 1 the gathered buffer already is Y.  Ragged shards (sizes differ by at most one row) are padded to the largest, gathered and trimmed.
    """
    M = Y_local.shape[0]
    counts = [r for _, r in plan]
    N = sum(counts)
    world = len(plan)
    if world == 1:
        return Y_local
    if len(set(counts)) == 1:
        buf = torch.empty((world * M, counts[0]), dtype=Y_local.dtype, device=Y_local.device)   # rank-major concat
        dist.all_gather_into_tensor(buf, Y_local.contiguous(), group=group)
        if M == 1:
            return buf.view(1, N)
        return buf.view(world, M, counts[0]).permute(1, 0, 2).reshape(M, N)
    cmax = max(counts)                      # ragged shards (differ by at most one row): pad, gather, trim
    padded = torch.zeros((M, cmax), dtype=Y_local.dtype, device=Y_local.device)
    padded[:, : Y_local.shape[1]] = Y_local
    buf = torch.empty((world * M, cmax), dtype=Y_local.dtype, device=Y_local.device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    buf = buf.view(world, M, cmax)
    return torch.cat([buf[r, :, : counts[r]] for r in range(world)], dim=1)


class NShardedLinear:
    """One (Wq, sw) pair sharded along N.  `compute(X, row0, rows) -> Y_local[M, rows]` is the rank-local
    product: on a GPU it calls w4a8_linear on the rank's shard; the CPU tests inject a host function."""

    def __init__(self, N, K, rank, world, shard_rows, compute, group=None):
        self.N, self.K, self.rank, self.world, self.group = N, K, rank, world, group
        self.plan = shard_plan(N, world, shard_rows)
        self.row0, self.rows = self.plan[rank]
        self.compute = compute

    def __call__(self, X):
        return all_gather_columns(self.compute(X, self.row0, self.rows), self.plan, self.group)


def expert_range(num_experts, rank, world):
    """Experts [base, base + count) of rank `rank`: equal contiguous blocks (num_experts must divide by world), the
    split w4a8_moe_block_shard expects (expert e's tensors start e - base experts into the rank's flat tensors)."""
    if num_experts % world != 0:
        raise ValueError("num_experts=%d is not a multiple of world=%d" % (num_experts, world))
    count = num_experts // world
    return rank * count, count


class ExpertShardedBlock:
    """Plain (collective) form of the expert-sharded routed-expert block, for comparison with the fused peer-store
    exchange of w4a8_moe_block_shard and for the CPU tests of the partition.

    `compute(n2, idx, base, count) -> so[nslots, H]` is the rank-local part: the down outputs of the slots whose expert
    lies in [base, base + count), zeros in every other row (on a GPU: the library's block on the rank's experts; the CPU
    tests inject the oracle).  Every row has exactly one owner, so an all-reduce(sum) of the zero-padded buffers IS the
    gather of the rows (x + 0 = x exactly); the combine then runs on every rank in the reference's fixed order
    (kernels/moe_fused.cuh:64,68-76): out[b] = sum over k ascending of dw[b,k] * so[b,k], each product rounded once."""

    def __init__(self, num_experts, topk, rank, world, compute, group=None):
        self.topk, self.group, self.compute = topk, group, compute
        self.base, self.count = expert_range(num_experts, rank, world)

    def __call__(self, n2, idx, dw):
        so = self.compute(n2, idx, self.base, self.count)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(so, op=dist.ReduceOp.SUM, group=self.group)
        S, H = n2.shape[0], so.shape[1]
        so = so.view(S, self.topk, H)
        w = dw.view(S, self.topk, 1).to(so.dtype)
        out = torch.zeros((S, H), dtype=so.dtype, device=so.device)
        for k in range(self.topk):
            out = out + w[:, k] * so[:, k]
        return out
