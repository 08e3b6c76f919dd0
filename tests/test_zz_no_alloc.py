"""lb_read_bwd_noalloc: the backward read for hosts that cannot allocate device memory.

Some callers of this library own no allocator they may use at call time -- a runtime that sizes all device memory at
start-up, a plugin host that hands over only the tensors of one call -- so they cannot provide the scratch rows that
lb_read_bwd wants. The variant keeps that scratch inside the library. This file checks, through the C ABI, that it
returns what lb_read_bwd returns (same kernels, so bit for bit), on two calls in a row (the built-in scratch keeps the
previous call's contents, which must not leak into the next result), and that it refuses rows wider than its limit.
It is named to be collected last: if it fails, every other test has already run.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _problem(L, n_tok, d, N, n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    code = L.dtype_code(dtype)
    V = (torch.randn(N, n_tok, d, device="cuda", generator=g) * 0.5).to(dtype)
    R = torch.rsqrt(V.float().pow(2).mean(-1) + 1e-6).contiguous()
    q = (torch.randn(d, device="cuda", generator=g) * 0.3).contiguous()
    dots = torch.einsum("ntd,d->nt", V.float(), q).contiguous()
    base = torch.randn(n_tok, d, device="cuda", generator=g).to(dtype)
    c0 = (torch.rand(n, device="cuda", generator=g) * 0.9 + 0.1).contiguous()
    cbar = (c0.view(1, -1) + 0.2 * torch.randn(n_tok, n, device="cuda", generator=g)).contiguous()
    out = torch.empty_like(base)
    tc, lg = torch.empty(n_tok, n, device="cuda"), torch.empty(n_tok, n, device="cuda")
    lse, lse0 = torch.empty(n_tok, device="cuda"), torch.empty(n_tok, device="cuda")
    L.check(L.lib().lb_read_fwd(L.ptr(V), L.ptr(R), L.ptr(dots), 0, L.ptr(base), L.ptr(cbar), L.ptr(c0), L.ptr(out),
                                L.ptr(tc), L.ptr(lg), L.ptr(lse), L.ptr(lse0), n_tok, d, N, n, code, L.stream_ptr()),
            "read forward")
    up = torch.randn(n_tok, d, device="cuda", generator=g).to(dtype)
    gt = torch.randn(n_tok, n, device="cuda", generator=g)
    return dict(V=V, R=R, q=q, cbar=cbar, c0=c0, lg=lg, lse=lse, lse0=lse0, g=up, gt=gt, code=code)


def _backward(L, pr, n_tok, d, N, n, accum, noalloc, dV0, dR0):
    dV, dR = dV0.clone(), dR0.clone()
    dcbar = torch.full((n_tok, n), float("nan"), device="cuda")
    dq = torch.full((d,), float("nan"), device="cuda")
    common = [L.ptr(pr["V"]), L.ptr(pr["R"]), L.ptr(dV), L.ptr(dR), L.ptr(pr["q"]), L.ptr(pr["g"]), L.ptr(pr["gt"]),
              L.ptr(pr["cbar"]), L.ptr(pr["c0"]), L.ptr(pr["lg"]), L.ptr(pr["lse"]), L.ptr(pr["lse0"]), L.ptr(dcbar),
              L.ptr(dq)]
    tail = [n_tok, d, N, n, int(accum), pr["code"], L.stream_ptr()]
    if noalloc:
        rc = L.lib().lb_read_bwd_noalloc(*common, *tail)
    else:
        scratch = torch.empty(L.lib().lb_read_bwd_scratch_bytes(d) // 4, device="cuda")
        rc = L.lib().lb_read_bwd(*common, L.ptr(scratch), *tail)
    L.check(rc, "read backward")
    torch.cuda.synchronize()
    return dq, dV, dR, dcbar


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_matches_read_bwd_twice_in_a_row(dtype):
    import loopback_b200._lib as L
    N = 6
    # two different problems back to back: the second call must not see anything of the first in the shared scratch
    # (the last problem runs at the widest row the entry point takes, LB_NOALLOC_MAX_D)
    for n_tok, d, n, accum, seed in ((300, 1024, 6, False, 1), (77, 768, 4, True, 2), (41, 3072, 5, True, 3)):
        pr = _problem(L, n_tok, d, N, n, dtype, seed)
        g = torch.Generator(device="cuda").manual_seed(100 + seed)
        dV0 = torch.randn(N, n_tok, d, device="cuda", generator=g).to(dtype)
        dR0 = torch.randn(N, n_tok, device="cuda", generator=g)
        want = _backward(L, pr, n_tok, d, N, n, accum, False, dV0, dR0)
        got = _backward(L, pr, n_tok, d, N, n, accum, True, dV0, dR0)
        again = _backward(L, pr, n_tok, d, N, n, accum, True, dV0, dR0)
        for a, b, c, name in zip(want, got, again, ("dq", "dV", "dR", "dcbar")):
            assert torch.isfinite(a.float()).all(), name
            assert torch.equal(a, b), f"{name}: no-alloc variant differs from lb_read_bwd"
            assert torch.equal(a, c), f"{name}: second call in a row differs"
    assert L.device_error() == 0


def test_noalloc_rejects_rows_beyond_its_limit():
    import loopback_b200._lib as L
    t = torch.zeros(8, 4096, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(8 * 4096, device="cuda")
    rc = L.lib().lb_read_bwd_noalloc(L.ptr(t), L.ptr(f), L.ptr(t), L.ptr(f), L.ptr(f), L.ptr(t), None, L.ptr(f),
                                     L.ptr(f), L.ptr(f), L.ptr(f), L.ptr(f), L.ptr(f), L.ptr(f), 8, 4096, 1, 1, 0,
                                     L.LB_DTYPE_BF16, None)
    assert rc == -3
    assert b"LB_NOALLOC_MAX_D" in L.lib().lb_last_error_string()
