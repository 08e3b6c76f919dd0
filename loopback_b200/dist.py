"""Multi-GPU plumbing of the read path: tokens shard across ranks, the query gradient is the only exchange.

Reads and writes are per-token, so a rank needs nothing from its peers in the forward; in the backward every rank
produces the gradient of the SAME (N - 1, d) query parameter from its own tokens, and the sum over ranks is the
gradient of the whole batch.  The reference gets that sum implicitly from FSDP's reduce-scatter of `query.grad`
(the query lives in the root FSDP unit, trainer/flame/models/parallelize_fla.py:549-554); here it is one explicit
fp32 all-reduce per pass.  The collective runs on whatever process group it is given (NCCL over NVLink on GPUs;
gloo in the CPU tests).

On the GPUs of one NVLink node the exchange can instead be the last backward's epilogue (`PeerQueryGrad`): the step
backwards write their query-gradient rows straight into a buffer the peers can address, and one small launch of this
library sums all ranks' buffers with plain peer loads -- no NCCL call, no launch and protocol latency on a 94 KB
message."""
from __future__ import annotations

import ctypes
import math
import os

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


def peer_slices(n_floats: int, flag_words: int, align: int = 64) -> tuple[int, int, int]:
    """Layout of a rank's peer-addressable allocation, in 4-byte words: (gradient words, flag offset, total words).
    The gradient is padded to whole 16-byte groups and the flag block starts on an `align`-word boundary."""
    if n_floats < 0 or flag_words <= 0:
        raise ValueError("sizes must be positive")
    grad = (n_floats + 3) // 4 * 4
    off = (grad + align - 1) // align * align
    return grad, off, off + flag_words


class PeerQueryGrad:
    """The query gradient of a pass, summed over the ranks of one node through peer memory (lb_peer_allreduce).

    `rows` is this rank's (N - 1, d) fp32 gradient buffer, allocated in symmetric memory so that every peer can read
    it: the step backwards write their rows into it. `reduce()` then launches the one-shot all-reduce on the current
    stream and returns the sum (identical bits on every rank: ranks are summed in rank order). Attach it to a stack
    (`stack.peer_reduce = PeerQueryGrad(...)`) and the pass's last backward does all of this itself: `query.grad`
    arrives already summed and the caller issues no collective.

    Construction is collective over `group` (a rendezvous and a barrier); afterwards no host synchronisation takes
    place, and the launch can be captured in a CUDA graph. The ranks' kernels wait on one another with bounded
    waits: a rank whose peer never arrives gets device error 6 (fused_dattn.device_error) instead of a hang. One
    rank per GPU; no multicast is used or set up."""

    def __init__(self, shape, device, group=None):
        from . import _lib
        import torch.distributed._symmetric_memory as symm
        if not dist.is_initialized():
            raise RuntimeError("PeerQueryGrad needs an initialised process group")
        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if self.world > _lib.LB_MAX_PEERS:
            raise RuntimeError(f"PeerQueryGrad serves at most {_lib.LB_MAX_PEERS} ranks (one NVLink node)")
        self.shape = tuple(int(x) for x in shape)
        self.n = math.prod(self.shape)
        self.n_pad, flag_off, total = peer_slices(self.n, int(_lib.lib().lb_peer_flag_words()))
        # plain peer loads only: keep torch from binding the allocation to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        dev = torch.device(device)
        self._mem = symm.empty(total, dtype=torch.float32, device=dev)
        self._hdl = symm.rendezvous(self._mem, group)
        self._mem.zero_()
        torch.cuda.synchronize(dev)
        dist.barrier(group=group)                 # every rank's flags are zero before any rank signals
        bases = [int(p) for p in self._hdl.buffer_ptrs]
        self._bufs = (ctypes.c_void_p * self.world)(*bases)
        self._flags = (ctypes.c_void_p * self.world)(*[b + 4 * flag_off for b in bases])
        self.rows = self._mem[:self.n].view(self.shape)
        self.device = dev

    def reduce(self, out: torch.Tensor | None = None) -> torch.Tensor:
        """Sum of every rank's `rows` (call once per pass, on every rank, after the rows are complete)."""
        from . import _lib
        buf = torch.empty(self.n_pad, device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().lb_peer_allreduce(self._bufs, self._flags, self.rank, self.world, _lib.ptr(buf),
                                                    self.n_pad, _lib.stream_ptr(self.device)), "peer all-reduce")
        res = buf[:self.n].view(self.shape)
        if out is not None:
            out.copy_(res)
            return out
        return res
