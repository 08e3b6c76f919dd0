"""Multi-GPU plumbing of the read path: tokens shard across ranks, the query gradient is the only exchange.

Reads and writes are per-token, so a rank needs nothing from its peers in the forward; in the backward every rank
produces the gradient of the SAME (N - 1, d) query parameter from its own tokens, and the sum over ranks is the
gradient of the whole batch.  The reference gets that sum implicitly from FSDP's reduce-scatter of `query.grad`
(the query lives in the root FSDP unit, trainer/flame/models/parallelize_fla.py:549-554); here it is one explicit
fp32 all-reduce per pass.  The collective runs on whatever process group it is given (NCCL over NVLink on GPUs;
gloo in the CPU tests)."""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_tokens(n_tok: int, rank: int, world: int) -> tuple[int, int]:
    """[start, stop) of the contiguous token range owned by `rank`: sizes differ by at most one, lower ranks first."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of size {world}")
    if n_tok < 0:
        raise ValueError("n_tok must be non-negative")
    base, extra = divmod(n_tok, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def allreduce_query_grad(grad: torch.Tensor, group=None, expected_shape=None, check: bool = True) -> torch.Tensor:
    """Sum the local query gradient over the ranks of `group`, in fp32, in place when `grad` is fp32.

    Every rank must pass the same shape. With `check` (the default) each rank contributes its shape, and whether it
    matches `expected_shape`, to a small all-gather first, and EVERY rank raises after that exchange if any of them
    disagrees -- none is left waiting in a collective its peer never joins. The exchange costs a host synchronisation
    per call; a training loop checks on its first pass and calls with check=False afterwards, which issues the
    all-reduce only."""
    if not dist.is_available() or not dist.is_initialized():
        return grad
    world = dist.get_world_size(group)
    if world == 1:
        return grad
    if check:
        ok = expected_shape is None or tuple(grad.shape) == tuple(expected_shape)
        rec = torch.tensor(list(grad.shape) + [0] * (4 - grad.dim()) + [1 if ok else 0], dtype=torch.int64,
                           device=grad.device)
        recs = [torch.empty_like(rec) for _ in range(world)]
        dist.all_gather(recs, rec, group=group)
        bad = [r for r, x in enumerate(recs) if int(x[4]) == 0]
        if bad:
            raise ValueError(f"query gradient shape differs from the expected {tuple(expected_shape)} on ranks {bad}: "
                             + str([x[:4].tolist() for x in recs]))
        if any(not torch.equal(x[:4], rec[:4]) for x in recs):
            raise RuntimeError("query gradient shapes differ across ranks: " + str([x[:4].tolist() for x in recs]))
    if grad.dtype == torch.float32:
        dist.all_reduce(grad, op=dist.ReduceOp.SUM, group=group)
        return grad
    buf = grad.float()
    dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
    grad.copy_(buf)
    return grad
