"""The one-shot all-reduce of the query gradient through peer memory (lb_peer_allreduce, dist.PeerQueryGrad).

On one GPU the ranks are emulated inside ONE launch: the "peers'" buffers and flag blocks are ordinary local
allocations, and the peers' flags are set beforehand, so the kernel waits for nobody (kernels that wait on one
another are never run as separate launches on one GPU). The bounded wait is tested the same way: a peer flag that
nothing sets, a short limit, and the kernel returns with the wait on record -- nothing traps, nothing hangs.

With two GPUs the real thing runs as two processes (this file is its own worker: `python -m torch.distributed.run
--nproc-per-node 2 tests/test_gpu_peer.py`): a whole pass whose last backward sums the query gradient over the ranks
is compared, bit for bit, with the rank-ordered sum of the ranks' local gradients."""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

pytestmark = pytest.mark.gpu
FAR = 0x3FFFFFFF            # an epoch no test reaches: a flag holding it never makes anyone wait


@pytest.fixture(scope="module")
def L():
    import loopback_b200._lib as lib
    lib.lib()
    return lib


def _blocks(L, world, n, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    bufs = [torch.randn(n, device="cuda", generator=g) for _ in range(world)]
    words = int(L.lib().lb_peer_flag_words())
    flags = [torch.zeros(words, device="cuda", dtype=torch.int32) for _ in range(world)]
    return bufs, flags, words


def _call(L, bufs, flags, rank, out):
    world = len(bufs)
    pb = (ctypes.c_void_p * world)(*[b.data_ptr() for b in bufs])
    pf = (ctypes.c_void_p * world)(*[f.data_ptr() for f in flags])
    return L.lib().lb_peer_allreduce(pb, pf, rank, world, L.ptr(out), out.numel(), L.stream_ptr())


@pytest.mark.parametrize("world,n", [(1, 64), (2, 23 * 1024), (4, 5 * 96), (8, 79 * 2048), (16, 4)])
def test_emulated_ranks_sum_in_rank_order(L, world, n):
    """The last rank of `world`, its peers' flags already at a far epoch: the sum over the buffers in rank order, call
    after call (the call counter lives on the device). A world of one is a copy."""
    bufs, flags, words = _blocks(L, world, n)
    me = world - 1
    ctas = words // (2 * 16 + 1)               # layout: [2 phases][LB_MAX_PEERS][ctas], then one counter per CTA
    f = flags[me].view(-1)
    for phase in range(2):
        for r in range(world):
            if r != me:
                base = (phase * 16 + r) * ctas
                f[base:base + ctas] = FAR
    want = bufs[0].clone()
    for r in range(1, world):
        want += bufs[r]
    for it in range(3):
        out = torch.full((n,), float("nan"), device="cuda")
        assert _call(L, bufs, flags, me, out) == 0
        assert L.device_error() == 0
        assert torch.equal(out, want)
        # what it told its peers: its epoch, in its own slot of both phases of every rank's block
        for r in range(world):
            fr = flags[r].view(-1)
            for phase in range(2):
                base = (phase * 16 + me) * ctas
                assert int(fr[base]) == it + 1
        bufs[0].mul_(1.5)
        want = bufs[0].clone()
        for r in range(1, world):
            want += bufs[r]


def test_a_peer_that_never_arrives_is_reported_not_waited_for(L):
    """A flag that nothing sets: with the limit at about a millisecond the kernel gives up, records code 6, writes no
    sum and returns; the next call with the flag set works."""
    n = 23 * 1024
    bufs, flags, words = _blocks(L, 2, n)
    ctas = words // (2 * 16 + 1)
    out = torch.full((n,), float("nan"), device="cuda")
    L.set_option("wait_cycles", 2_000_000)
    try:
        assert _call(L, bufs, flags, 0, out) == 0
        torch.cuda.synchronize()
    finally:
        L.reset_options()
    assert L.device_error(clear=True) == 6
    assert torch.isnan(out).all(), "a rank that gave up writes no sum"
    f = flags[0].view(-1)
    for phase in range(2):
        base = (phase * 16 + 1) * ctas
        f[base:base + ctas] = FAR
    assert _call(L, bufs, flags, 0, out) == 0
    assert L.device_error() == 0
    assert torch.equal(out, bufs[0] + bufs[1])


def test_arguments(L):
    bufs, flags, _ = _blocks(L, 2, 16)
    out = torch.empty(16, device="cuda")
    lib = L.lib()
    pb = (ctypes.c_void_p * 2)(*[b.data_ptr() for b in bufs])
    pf = (ctypes.c_void_p * 2)(*[f.data_ptr() for f in flags])
    s = L.stream_ptr()
    assert lib.lb_peer_allreduce(pb, pf, 2, 2, L.ptr(out), 16, s) == -1      # rank outside the world
    assert lib.lb_peer_allreduce(pb, pf, 0, 17, L.ptr(out), 16, s) == -1     # more ranks than LB_MAX_PEERS
    assert lib.lb_peer_allreduce(pb, pf, 0, 2, L.ptr(out), 6, s) == -1       # not whole 16-byte groups
    assert lib.lb_peer_allreduce(pb, pf, 0, 2, None, 16, s) == -1
    assert lib.lb_peer_allreduce(pb, pf, 0, 2, L.ptr(out), 0, s) == 0        # nothing to do
    pb[1] = None
    assert lib.lb_peer_allreduce(pb, pf, 0, 2, L.ptr(out), 16, s) == -1
    pb[1] = bufs[1].data_ptr() + 4
    assert lib.lb_peer_allreduce(pb, pf, 0, 2, L.ptr(out), 16, s) == -2      # misaligned peer buffer
    assert L.device_error() == 0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_on_two_gpus():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TORCH_SYMM_MEM_DISABLE_MULTICAST="1")
    port = 29500 + os.getpid() % 2000
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.abspath(__file__)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "PEER-OK" in res.stdout


def _worker():
    """One rank of the two-GPU test: a small pass with the peer reduction against the same pass without it."""
    import torch.distributed as dist
    from loopback_b200 import fused_dattn as FD
    from loopback_b200.cell import LoopDeltaAttnRes

    rank, local = int(os.environ["RANK"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    world = dist.get_world_size()
    d, K, Rr, b, t = 512, 3, 2, 2, 700 + 40 * rank        # ranks hold different numbers of tokens
    N = K * Rr
    cell = LoopDeltaAttnRes(d, Rr, K, beta=0.75).to(dev)
    g = torch.Generator(device=dev).manual_seed(1)
    with torch.no_grad():
        cell.query.copy_(torch.randn(N - 1, d, device=dev, generator=g) * 0.05)   # same parameter on every rank
    g.manual_seed(100 + rank)
    h0 = torch.randn(b, t, d, device=dev, generator=g).bfloat16().requires_grad_(True)
    D = [(torch.randn(b, t, d, device=dev, generator=g) * 0.3).bfloat16() for _ in range(N)]
    G = [torch.randn(b, t, d, device=dev, generator=g).bfloat16() for _ in range(N)]

    def one_pass():
        cell.query.grad = None
        h0.grad = None
        stack = cell.new_stack((b, t, d), torch.bfloat16, dev, scores=True)
        x, deltas, keys, coeffs, prior, outs = h0, [], [], None, None, []
        for s in range(N):
            l, blk = divmod(s, K)
            hs = x + D[s]
            deltas.append(stack.write(s, hs, x))
            x, coeffs, prior = cell.combine(hs, h0, deltas, coeffs, prior, l, blk, keys=keys, stack=stack)
            outs.append(x)
        torch.autograd.backward(outs, G)
        return cell.query.grad.clone(), h0.grad.clone()

    local_dq, local_dh0 = one_pass()
    parts = [torch.empty_like(local_dq) for _ in range(world)]
    dist.all_gather(parts, local_dq)
    want = parts[0].clone()
    for r in range(1, world):
        want += parts[r]

    cell.enable_peer_reduce(dev)
    for it in range(3):
        dq, dh0 = one_pass()
        assert FD.device_error() == 0, f"rank {rank}: a bounded wait ran out"
        assert torch.equal(dq, want), f"rank {rank} pass {it}: peer sum differs from the rank-ordered sum"
        assert torch.equal(dh0, local_dh0)

    # the same pass as a CUDA graph (the call counter lives on the device: a replay is a new call)
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        one_pass()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    dist.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        cell.query.grad = None
        dq_g, _ = one_pass()
    for it in range(3):
        graph.replay()
        torch.cuda.synchronize()
        assert FD.device_error() == 0
        assert torch.equal(dq_g, want), f"rank {rank} replay {it}"
    dist.barrier()
    if rank == 0:
        print("PEER-OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    _worker()
