"""CPU-side checks: the C-ABI library loads and exports what the header declares, argument validation needs no GPU,
the token sharding and the query-gradient exchange work across two gloo ranks."""
import ctypes
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "loopback_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    import loopback_b200._lib as L
    if not os.path.exists(L.LIB_PATH):
        from loopback_b200 import build
        build.build()
    handle = ctypes.CDLL(L.LIB_PATH)
    declared = header_symbols()
    assert len(declared) >= 13
    for name in declared:
        assert hasattr(handle, name), f"{name} is declared in include/loopback_b200.h but not exported"
    assert set(declared) == set(L.SYMBOLS), "the ctypes table and the header disagree"
    assert L.lib().lb_version() == 1


def test_argument_validation_needs_no_gpu():
    import loopback_b200._lib as L
    lib = L.lib()
    assert lib.lb_rstd_fwd(None, None, 4, 64, 1e-6, L.LB_DTYPE_BF16, None) == -1
    assert b"NULL" in lib.lb_last_error_string()
    assert lib.lb_rstd_fwd(None, None, 4, 63, 1e-6, L.LB_DTYPE_BF16, None) == -2
    assert lib.lb_rstd_fwd(None, None, 4, 64, 1e-6, 9, None) == -1
    assert lib.lb_rstd_fwd(None, None, 4, 1 << 20, 1e-6, L.LB_DTYPE_F32, None) == -3
    assert lib.lb_set_option(b"no_such_knob", 1) == -1
    assert lib.lb_read_bwd_scratch_bytes(1024) >= 148 * 1024 * 4
    with pytest.raises(RuntimeError):
        L.dtype_code(torch.float64)


def test_no_cpu_path():
    """CPU tensors are refused loudly: there is no eager or CPU fallback behind the entry points."""
    import loopback_b200.fused_dattn as FD
    from loopback_b200.cell import LoopDeltaAttnRes
    with pytest.raises(RuntimeError):
        FD.rstd(torch.zeros(2, 3, 64), 1e-6)
    with pytest.raises(RuntimeError):
        FD.DattnStack(4, (1, 2, 64), torch.float32, "cpu")
    x = torch.zeros(1, 2, 64)
    assert FD.fused_read_supported(x, [x], [torch.ones(1, 2, 1)], torch.ones(1, 2, 1)) is False
    cell = LoopDeltaAttnRes(64, 2, 2)
    assert cell.query.shape == (3, 64) and float(cell.query.detach().abs().max()) == 0.0
    with pytest.raises(RuntimeError):
        cell.combine(x, x, [x, x], torch.ones(1, 2, 1), torch.ones(1), 0, 1)
    with pytest.raises(ValueError):
        LoopDeltaAttnRes(64, 0, 2)
    with pytest.raises(ValueError):
        LoopDeltaAttnRes(64, 2, 2, beta=1.0)


def test_shard_tokens():
    from loopback_b200.dist import shard_tokens
    for n_tok in (0, 1, 7, 64, 32768, 262144 + 3):
        for world in (1, 2, 3, 8):
            spans = [shard_tokens(n_tok, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n_tok
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_tokens(8, 2, 2)


def test_peer_allocation_layout():
    """A rank's peer-addressable allocation: the gradient padded to whole 16-byte groups, then the flag block on a
    256-byte boundary; the flag block's size comes from the library (no GPU needed to ask)."""
    from loopback_b200.dist import peer_slices
    from loopback_b200 import _lib
    words = int(_lib.lib().lb_peer_flag_words())
    assert words == 2 * _lib.LB_MAX_PEERS * 32 + 32
    for n in (0, 1, 4, 23 * 1024, 79 * 2048 + 2):
        grad, off, total = peer_slices(n, words)
        assert grad % 4 == 0 and 0 <= grad - n < 4
        assert off % 64 == 0 and off >= grad and total == off + words
    with pytest.raises(ValueError):
        peer_slices(-1, words)


def test_peer_reduce_needs_a_process_group():
    from loopback_b200.cell import LoopDeltaAttnRes
    cell = LoopDeltaAttnRes(64, 2, 2)
    assert cell.peer_reduce is None and "peer_reduce" not in cell.state_dict()
    with pytest.raises(RuntimeError):
        cell.enable_peer_reduce("cuda")


WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, sys.argv[1])
from loopback_b200.dist import allreduce_query_grad, shard_tokens
from oracle import c_oracle as CO
import numpy as np
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
mode = sys.argv[2]
if mode == "sum":
    # the query gradient of the whole batch is the sum of the shards' gradients (checked with the CPU oracle)
    K, R, n_tok, d = 2, 2, 12, 64
    N = K * R
    rng = np.random.default_rng(0)
    h0 = rng.standard_normal((n_tok, d)); D = rng.standard_normal((N, n_tok, d)) * 0.5
    Q = rng.standard_normal((N - 1, d)) * 0.3; G = rng.standard_normal((N, n_tok, d))
    full = CO.chain(h0, D, Q, G, K, R, 0.75, 1e-6, False)["dq"]
    a, b = shard_tokens(n_tok, rank, world)
    mine = CO.chain(np.ascontiguousarray(h0[a:b]), np.ascontiguousarray(D[:, a:b]), Q, np.ascontiguousarray(G[:, a:b]),
                    K, R, 0.75, 1e-6, False)["dq"]
    g = torch.from_numpy(mine).float()
    allreduce_query_grad(g, expected_shape=(N - 1, d))
    err = float((g.double() - torch.from_numpy(full)).abs().max() / np.abs(full).max())
    assert err < 1e-5, err
    gb = torch.from_numpy(mine).bfloat16()
    allreduce_query_grad(gb)
    assert float((gb.double() - torch.from_numpy(full)).abs().max() / np.abs(full).max()) < 2e-2
elif mode == "mismatch":
    g = torch.zeros(3 + rank, 8)
    try:
        allreduce_query_grad(g)
    except RuntimeError as e:
        assert "differ" in str(e)
    else:
        raise SystemExit("a shape mismatch across ranks went undetected")
elif mode == "expected":
    # one rank holds a gradient of the wrong shape: BOTH ranks raise, after the exchange, and neither is left waiting
    g = torch.zeros(3, 8) if rank == 0 else torch.zeros(4, 8)
    try:
        allreduce_query_grad(g, expected_shape=(3, 8))
    except ValueError as e:
        assert "ranks [1]" in str(e), str(e)
    else:
        raise SystemExit("a wrong shape on a peer went undetected")
    # check=False: the all-reduce alone
    g2 = torch.full((3, 8), float(rank + 1))
    allreduce_query_grad(g2, check=False)
    assert float(g2[0, 0]) == 3.0
elif mode == "raise":
    # a rank that fails before the exchange: the survivor's collective ends with an error instead of hanging
    if rank == 1:
        raise SystemExit(3)
    try:
        allreduce_query_grad(torch.zeros(3, 8))
    except Exception:
        raise SystemExit(0)
    raise SystemExit("the collective returned although the peer had left")
dist.destroy_process_group()
"""


def _spawn(mode, world=2, expect=(0, 0), timeout=120):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="2", GLOO_SOCKET_IFNAME="lo")
        procs.append(subprocess.Popen([sys.executable, "-c", WORKER, ROOT, mode], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=timeout)[0] for p in procs]
    codes = tuple(p.returncode for p in procs)
    assert codes == expect, (codes, outs)


def test_query_grad_allreduce_two_gloo_ranks():
    _spawn("sum")


def test_shape_mismatch_is_detected_on_every_rank():
    _spawn("mismatch")


def test_unexpected_shape_on_one_rank_raises_on_all():
    _spawn("expected")


def test_rank_failure_does_not_hang_the_survivor():
    _spawn("raise", expect=(0, 3))
