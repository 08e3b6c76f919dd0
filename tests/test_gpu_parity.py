"""Parity of the CUDA path with the CPU oracle and with tensors of the unmodified reference (tests/golden/).

Every test here needs a B200 and calls the kernels through the C ABI (directly, or through the `fused_dattn`
drop-in module that binds it). Tolerances: fp32 <= 1e-5 relative (max-abs error / max-abs reference) on every output
and gradient; bf16 storage <= 2e-2 * RMS(out) max-abs per read, teacher-forced, against the read evaluated in fp32 on
the same bf16-rounded inputs; bf16 gradients err <= 2 * err_reference + 2e-3, both against an fp64 evaluation.
"""
import ctypes
import os

import numpy as np
import pytest
import torch

import cases
from oracle import c_oracle as CO
from oracle import torch_oracle as TO

pytestmark = pytest.mark.gpu

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL32 = 1e-5


def rel(a, b):
    a = a.detach().double().cpu() if torch.is_tensor(a) else torch.as_tensor(np.asarray(a, np.float64))
    b = b.detach().double().cpu() if torch.is_tensor(b) else torch.as_tensor(np.asarray(b, np.float64))
    return float((a - b).abs().max() / b.abs().max().clamp_min(1e-30))


@pytest.fixture(scope="module")
def FD():
    import loopback_b200.fused_dattn as fd
    yield fd
    assert fd.device_error() == 0, "a kernel gave up a bounded wait"


@pytest.fixture(scope="module")
def L():
    import loopback_b200._lib as lib
    return lib


@pytest.fixture(autouse=True)
def _default_kernel_choice(L):
    """A test that forces a kernel through lb_set_option leaves the choice by size behind, pass or fail."""
    yield
    L.reset_options()


def cuda(x):
    return x.cuda() if torch.is_tensor(x) else x


# ------------------------------------------------------------------------------------------------------------
# 1. the write, through the C ABI
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
# 0: by size (one CTA per token for small batches, the tensor-core kernel for large bf16 ones); 1, 2: the tiled kernel;
# 3: the tensor-core kernel whatever the size (bf16 only; fp32 rows keep the choice by size)
@pytest.mark.parametrize("tile", [0, 1, 2, 3])
@pytest.mark.parametrize("n_tok,d,N", [(5, 64, 6), (37, 768, 6), (130, 1024, 6), (33, 1536, 6), (9, 3072, 6),
                                       (64, 2048, 6), (19, 512, 70), (5000, 320, 6), (40000, 136, 4),
                                       (300, 4096, 3), (700, 1024, 40)])
@pytest.mark.parametrize("q_in_bf16", [False, True])
def test_write_matches_oracle(L, dtype, n_tok, d, N, tile, q_in_bf16):
    """q_in_bf16: queries that are exact in bf16 (a bf16 parameter): the tensor-core kernel then needs one of its
    three query terms only, and finds that out by itself."""
    if q_in_bf16 and not (tile == 3 and dtype == torch.bfloat16):
        pytest.skip("only the tensor-core kernel treats bf16-exact queries specially")
    NQ = N - 1
    L.set_option("write_tt", tile)
    g = torch.Generator().manual_seed(n_tok * 7 + d)
    x = torch.randn(n_tok, d, generator=g).to(dtype)
    Q = torch.randn(NQ, d, generator=g) * 0.3
    if q_in_bf16:
        Q = Q.bfloat16().float()
    code = L.dtype_code(dtype)
    V = torch.zeros(N, n_tok, d, dtype=dtype, device="cuda")
    R = torch.zeros(N, n_tok, device="cuda")
    DOTS = torch.full((NQ, N, n_tok), float("nan"), device="cuda")
    xc, Qc = x.cuda(), Q.cuda()
    hs = []
    for s in range(N):
        h = (x.float() + torch.randn(n_tok, d, generator=g) * 0.5).to(dtype)
        hs.append(h)
        hc = h.cuda()
        L.check(L.lib().lb_write(L.ptr(hc), L.ptr(xc), L.ptr(V), L.ptr(R), L.ptr(Qc), L.ptr(DOTS), n_tok, d, N, NQ, s,
                                 1e-6, code, L.stream_ptr()), "write")
    torch.cuda.synchronize()
    L.set_option("write_tt", 0)
    for s in range(N):
        v_ref, r_ref = CO.write(hs[s].float().numpy(), x.float().numpy(), 1e-6, dtype == torch.bfloat16)
        assert torch.equal(V[s].float().cpu(), torch.from_numpy(v_ref)), "the stored update must be bit-exact"
        assert rel(R[s], r_ref) < TOL32
        j0 = max(s - 1, 0)
        want = torch.from_numpy(v_ref).double() @ Q.double().t()          # [n_tok, NQ]
        got = DOTS[:, s, :].t().cpu()
        assert rel(got[:, j0:], want[:, j0:]) < TOL32
        assert torch.isnan(got[:, :j0]).all(), "queries that never read update s must not be scored"


def test_write_rejects_bad_arguments(L):
    t = torch.zeros(4, 64, device="cuda")
    lib = L.lib()
    assert lib.lb_write(None, L.ptr(t), L.ptr(t), None, None, None, 4, 64, 2, 1, 0, 1e-6, 0, None) == -1
    assert lib.lb_write(L.ptr(t), L.ptr(t), L.ptr(t), None, None, None, 4, 64, 2, 1, 5, 1e-6, 0, None) == -1
    assert lib.lb_write(L.ptr(t), L.ptr(t), L.ptr(t), None, None, None, 4, 63, 2, 1, 0, 1e-6, 1, None) == -2
    assert lib.lb_write(L.ptr(t), L.ptr(t), L.ptr(t), None, None, None, 4, 64, 2, 1, 0, 1e-6, 7, None) == -1
    assert b"dtype" in lib.lb_last_error_string()
    assert lib.lb_read_fwd(L.ptr(t), L.ptr(t), L.ptr(t), 0, L.ptr(t), L.ptr(t), L.ptr(t), L.ptr(t), L.ptr(t), None,
                           None, None, 4, 64, 200, 129, 0, None) == -3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_tok,d,n,accum", [(70, 1024, 5, True), (33, 1536, 3, False), (9, 3072, 4, True),
                                             (130, 768, 2, True), (5, 64, 6, False), (64, 2048, 7, True)])
def test_read_bwd_final_equals_the_three_separate_kernels(L, dtype, n_tok, d, n, accum):
    """lb_read_bwd_final == lb_read_bwd, then lb_rstd_bwd_acc on the newest update, then lb_write_bwd_dx: bit for bit."""
    N = 8
    g = torch.Generator(device="cuda").manual_seed(n_tok + d + n)
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
                                L.ptr(tc), L.ptr(lg), L.ptr(lse), L.ptr(lse0), n_tok, d, N, n, code, L.stream_ptr()), "fwd")
    up = torch.randn(n_tok, d, device="cuda", generator=g).to(dtype)
    gt = torch.randn(n_tok, n, device="cuda", generator=g)
    dV0 = torch.randn(N, n_tok, d, device="cuda", generator=g).to(dtype)
    dR0 = torch.randn(N, n_tok, device="cuda", generator=g)
    scratch = torch.empty(L.lib().lb_read_bwd_scratch_bytes(d) // 4, device="cuda")

    def args(dV, dR, dcbar, dq):
        return [L.ptr(V), L.ptr(R), L.ptr(dV), L.ptr(dR), L.ptr(q), L.ptr(up), L.ptr(gt), L.ptr(cbar), L.ptr(c0),
                L.ptr(lg), L.ptr(lse), L.ptr(lse0), L.ptr(dcbar), L.ptr(dq), L.ptr(scratch)]
    tail = [n_tok, d, N, n, int(accum), code, L.stream_ptr()]
    dV1, dR1 = dV0.clone(), dR0.clone()
    dcb1, dq1 = torch.empty(n_tok, n, device="cuda"), torch.empty(d, device="cuda")
    L.check(L.lib().lb_read_bwd(*args(dV1, dR1, dcb1, dq1), *tail), "bwd")
    L.check(L.lib().lb_rstd_bwd_acc(L.ptr(V[n - 1]), L.ptr(R[n - 1]), L.ptr(dR1[n - 1]), L.ptr(dV1[n - 1]), n_tok, d, code,
                                    L.stream_ptr()), "rstd acc")
    neg1 = torch.empty(n_tok, d, device="cuda", dtype=dtype)
    L.check(L.lib().lb_write_bwd_dx(L.ptr(dV1[n - 1]), L.ptr(neg1), n_tok * d, code, L.stream_ptr()), "neg")
    dV2, dR2 = dV0.clone(), dR0.clone()
    dcb2, dq2 = torch.empty(n_tok, n, device="cuda"), torch.empty(d, device="cuda")
    neg2 = torch.full((n_tok, d), float("nan"), device="cuda", dtype=dtype)
    L.check(L.lib().lb_read_bwd_final(*args(dV2, dR2, dcb2, dq2), L.ptr(neg2), *tail), "bwd final")
    torch.cuda.synchronize()
    assert torch.equal(dV1[:n], dV2[:n]) and torch.equal(dR1[:n], dR2[:n])
    assert torch.equal(dV1[n:], dV2[n:]), "slices beyond n must not be touched"
    assert torch.equal(dcb1, dcb2) and torch.equal(dq1, dq2) and torch.equal(neg1, neg2)
    assert L.device_error() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_tok,d,n,accum,blend", [(70, 1024, 5, True, True), (33, 1536, 3, False, True),
                                                   (9, 3072, 4, True, False), (130, 768, 2, True, True),
                                                   (5, 64, 6, False, False), (64, 2048, 7, True, True),
                                                   (300, 320, 9, True, True)])
def test_step_bwd_equals_combine_bwd_plus_the_torch_glue(L, dtype, n_tok, d, n, accum, blend):
    """lb_step_bwd == lb_combine_bwd (finalising) followed by what autograd does around it: dx is the negated
    gradient of the update, dh that gradient plus the base's (g, or g - beta g at an iteration's end), dh0 the
    accumulated beta g. Bit for bit, in the storage dtype's arithmetic."""
    N, beta, lam = 10, 0.75, 0.25 if blend else 1.0
    g = torch.Generator(device="cuda").manual_seed(3 * n_tok + d + n)
    code = L.dtype_code(dtype)
    V = (torch.randn(N, n_tok, d, device="cuda", generator=g) * 0.5).to(dtype)
    R = torch.rsqrt(V.float().pow(2).mean(-1) + 1e-6).contiguous()
    q = (torch.randn(d, device="cuda", generator=g) * 0.3).contiguous()
    dots = torch.einsum("ntd,d->nt", V.float(), q).contiguous()
    prop = torch.randn(n_tok, d, device="cuda", generator=g).to(dtype)
    h0 = torch.randn(n_tok, d, device="cuda", generator=g).to(dtype)
    c0 = (torch.rand(n, device="cuda", generator=g) * 0.9 + 0.1).contiguous()
    tcp = (c0[:n - 1].view(1, -1) + 0.2 * torch.randn(n_tok, n - 1, device="cuda", generator=g)).contiguous()
    out = torch.empty_like(prop)
    tc, lg = torch.empty(n_tok, n, device="cuda"), torch.empty(n_tok, n, device="cuda")
    lse, lse0 = torch.empty(n_tok, device="cuda"), torch.empty(n_tok, device="cuda")
    L.check(L.lib().lb_combine_fwd(L.ptr(V), L.ptr(R), L.ptr(dots), 0, L.ptr(prop), L.ptr(h0) if blend else None, beta,
                                   L.ptr(tcp), lam, L.ptr(c0), L.ptr(out), L.ptr(tc), L.ptr(lg), L.ptr(lse), L.ptr(lse0),
                                   n_tok, d, N, n, code, L.stream_ptr()), "fwd")
    up = torch.randn(n_tok, d, device="cuda", generator=g).to(dtype)
    gt = torch.randn(n_tok, n, device="cuda", generator=g)
    dV0 = torch.randn(N, n_tok, d, device="cuda", generator=g).to(dtype)
    dR0 = torch.randn(N, n_tok, device="cuda", generator=g)
    dh0_0 = torch.randn(n_tok, d, device="cuda", generator=g).to(dtype)
    scratch = torch.empty(L.lib().lb_read_bwd_scratch_bytes(d) // 4, device="cuda")
    head = [L.ptr(V), L.ptr(R)]
    mid = [L.ptr(q), L.ptr(up), L.ptr(gt), L.ptr(tcp), lam, L.ptr(c0), L.ptr(lg), L.ptr(lse), L.ptr(lse0)]
    tail = [n_tok, d, N, n, int(accum), code, L.stream_ptr()]
    dV1, dR1 = dV0.clone(), dR0.clone()
    dtc1, dq1 = torch.empty(n_tok, n - 1, device="cuda"), torch.empty(d, device="cuda")
    neg1 = torch.empty(n_tok, d, device="cuda", dtype=dtype)
    L.check(L.lib().lb_combine_bwd(*head, L.ptr(dV1), L.ptr(dR1), *mid, L.ptr(dtc1), L.ptr(dq1), L.ptr(scratch),
                                   L.ptr(neg1), 1, *tail), "combine backward")
    for dh0_accum in ((False, True) if blend else (False,)):
        dV2, dR2 = dV0.clone(), dR0.clone()
        dtc2, dq2 = torch.empty(n_tok, n - 1, device="cuda"), torch.empty(d, device="cuda")
        dh = torch.full((n_tok, d), float("nan"), device="cuda", dtype=dtype)
        dx = torch.full((n_tok, d), float("nan"), device="cuda", dtype=dtype)
        dh0 = dh0_0.clone() if dh0_accum else torch.full((n_tok, d), float("nan"), device="cuda", dtype=dtype)
        L.check(L.lib().lb_step_bwd(*head, L.ptr(dV2), L.ptr(dR2), *mid, L.ptr(dtc2), L.ptr(dq2), L.ptr(scratch),
                                    L.ptr(dh), L.ptr(dx), L.ptr(dh0) if blend else None, int(dh0_accum), int(blend), beta,
                                    *tail), "step backward")
        torch.cuda.synchronize()
        assert torch.equal(dV1[:n - 1], dV2[:n - 1]) and torch.equal(dR1[:n], dR2[:n])
        assert torch.equal(dV2[n - 1:], dV0[n - 1:]), "the finished update's gradient is handed out, not stored"
        assert torch.equal(dtc1, dtc2) and torch.equal(dq1, dq2) and torch.equal(dx, neg1)
        if blend:
            bg = up * beta
            assert torch.equal(dh, dV1[n - 1] + (up - bg))
            assert torch.equal(dh0, dh0_0 + bg if dh0_accum else bg)
        else:
            assert torch.equal(dh, dV1[n - 1] + up)
    assert L.device_error() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_tok,d,N,s,blend", [(64, 2048, 80, 79, True), (64, 2048, 80, 40, False), (5, 64, 6, 1, False),
                                               (37, 768, 12, 5, True), (130, 1024, 24, 23, True), (9, 3072, 8, 3, False),
                                               (3, 4096, 6, 4, True), (300, 320, 10, 9, False), (17, 136, 130, 127, True)])
def test_step_fwd_equals_write_then_read(L, dtype, n_tok, d, N, s, blend):
    """lb_step_fwd (one launch, no cached scores, two sweeps over L2) against lb_write followed by lb_combine_fwd: the
    stored update bit for bit, its key scale, the coefficients and the saved softmax statistics to fp32 round-off,
    the output to fp32 round-off (fp32 rows) or the last bf16 bit; and the zero-query identity bit for bit."""
    n, NQ, beta, lam = s + 1, N - 1, 0.75, 0.25 if blend else 1.0
    g = torch.Generator(device="cuda").manual_seed(n_tok + d + s)
    code = L.dtype_code(dtype)
    V = (torch.randn(N, n_tok, d, device="cuda", generator=g) * 0.5).to(dtype)
    R = torch.rsqrt(V.float().pow(2).mean(-1) + 1e-6).contiguous()
    h, x, h0 = (torch.randn(n_tok, d, device="cuda", generator=g).to(dtype) for _ in range(3))
    c0 = (torch.rand(n, device="cuda", generator=g) * 0.9 + 0.1).contiguous()
    tcp = (c0[:n - 1].view(1, -1) + 0.2 * torch.randn(n_tok, n - 1, device="cuda", generator=g)).contiguous()
    for zero_query in (False, True):
        Q = torch.zeros(NQ, d, device="cuda") if zero_query else torch.randn(NQ, d, device="cuda", generator=g) * 0.3
        tcp_ = (c0[:n - 1] / lam).view(1, -1).expand(n_tok, -1).contiguous() if zero_query else tcp
        c0_ = (lam * torch.cat((c0[:n - 1] / lam, torch.ones(1, device="cuda")))).contiguous() if zero_query else c0
        # reference: the two launches, scores cached by the writes
        V1, R1 = V.clone(), R.clone()
        DOTS = torch.einsum("ntd,qd->qnt", V1.float(), Q).contiguous()
        L.check(L.lib().lb_write(L.ptr(h), L.ptr(x), L.ptr(V1), L.ptr(R1), L.ptr(Q), L.ptr(DOTS), n_tok, d, N, NQ, s, 1e-6,
                                 code, L.stream_ptr()), "write")
        out1 = torch.empty_like(h)
        tc1, lg1 = torch.empty(n_tok, n, device="cuda"), torch.empty(n_tok, n, device="cuda")
        lse1, lse01 = torch.empty(n_tok, device="cuda"), torch.empty(n_tok, device="cuda")
        L.check(L.lib().lb_combine_fwd(L.ptr(V1), L.ptr(R1), L.ptr(DOTS), s - 1, L.ptr(h), L.ptr(h0) if blend else None,
                                       beta, L.ptr(tcp_), lam, L.ptr(c0_), L.ptr(out1), L.ptr(tc1), L.ptr(lg1),
                                       L.ptr(lse1), L.ptr(lse01), n_tok, d, N, n, code, L.stream_ptr()), "combine forward")
        V2, R2 = V.clone(), R.clone()
        out2 = torch.full_like(h, float("nan"))
        tc2, lg2 = torch.full((n_tok, n), float("nan"), device="cuda"), torch.empty(n_tok, n, device="cuda")
        lse2, lse02 = torch.empty(n_tok, device="cuda"), torch.empty(n_tok, device="cuda")
        L.check(L.lib().lb_step_fwd(L.ptr(h), L.ptr(x), L.ptr(h0) if blend else None, beta, L.ptr(V2), L.ptr(R2), L.ptr(Q),
                                    L.ptr(tcp_), lam, L.ptr(c0_), L.ptr(out2), L.ptr(tc2), L.ptr(lg2), L.ptr(lse2),
                                    L.ptr(lse02), n_tok, d, N, s, 1e-6, code, L.stream_ptr()), "step forward")
        torch.cuda.synchronize()
        assert torch.equal(V1, V2), "the stored update must be bit-exact, and no other slice touched"
        assert rel(R2[s], R1[s]) < 1e-6 and torch.equal(R2[:s], R1[:s])
        if zero_query:
            base = h + beta * (h0 - h) if blend else h
            assert torch.equal(out2, base) and torch.equal(tc2, c0_.view(1, -1).expand(n_tok, -1))
            continue
        assert rel(tc2, tc1) < TOL32 and rel(lg2, lg1) < TOL32
        assert rel(lse2, lse1) < TOL32 and rel(lse02, lse01) < TOL32
        if dtype == torch.float32:
            assert rel(out2, out1) < TOL32
        else:
            diff = (out2.float() - out1.float()).abs()
            ulp = out1.float().abs().clamp_min(1e-3) * 2.0 ** -7
            assert bool((diff <= ulp).all()), "bf16 outputs may differ in the last bit only"
            assert float((diff > 0).float().mean()) < 0.05
    assert L.device_error() == 0


# ------------------------------------------------------------------------------------------------------------
# 2. one read, list layout, in the style of the reference's kernel test (tests/test_fused_dattn.py:48-108)
# ------------------------------------------------------------------------------------------------------------
def run_read_gpu(FD, deltas, proposal, h0, q, prior, coeffs, up, up2, boundary, beta=0.75):
    deltas = [x.detach().clone().cuda().requires_grad_() for x in deltas]
    proposal = proposal.detach().clone().cuda().requires_grad_()
    h0 = h0.detach().clone().cuda().requires_grad_()
    cf = coeffs.detach().clone().cuda().requires_grad_()
    qq = q.detach().clone().cuda().float().requires_grad_()
    base = proposal + beta * (h0 - proposal) if boundary else proposal
    ones = torch.ones(*proposal.shape[:-1], 1, device="cuda")
    cbar = torch.cat((cf, ones), dim=-1)
    c0 = torch.cat((prior.cuda(), torch.ones(1, device="cuda")), dim=-1)
    if boundary:
        cbar, c0 = (1.0 - beta) * cbar, (1.0 - beta) * c0
    rstds = [FD.rstd(x, 1e-6) for x in deltas]
    assert FD.fused_read_supported(base, deltas, rstds, cbar)
    out, tc = FD.FusedDattnRead.apply(qq, base, cbar, c0, *deltas, *rstds)
    ((out.float() * up.cuda()).sum() + (tc * up2.cuda()).sum()).backward()
    zero = torch.zeros_like(proposal)
    return dict(out=out.detach(), tc=tc.detach(), dq=qq.grad, dd=torch.stack([x.grad for x in deltas]),
                dprop=proposal.grad, dh0=h0.grad if h0.grad is not None else zero, dcoef=cf.grad)


def run_read_oracle(deltas, proposal, h0, q, prior, coeffs, up, up2, boundary, hi, accumulate, beta=0.75):
    dl = [x.detach().to(hi).clone().requires_grad_() for x in deltas]
    pr, hh = (x.detach().to(hi).clone().requires_grad_() for x in (proposal, h0))
    ct = torch.float64 if hi == torch.float64 else torch.float32
    cf = coeffs.detach().to(ct).clone().requires_grad_()
    qq = q.detach().to(ct).clone().requires_grad_()
    base, cbar, c0 = TO.prologue(pr, hh, cf, prior.to(ct), beta, boundary)
    out, tc = TO.read(base, dl, qq, cbar, c0, 1e-6, accumulate=accumulate)
    ((out.to(ct) * up.to(ct)).sum() + (tc * up2.to(ct)).sum()).backward()
    zero = torch.zeros_like(pr)
    return dict(out=out.detach(), tc=tc.detach(), dq=qq.grad, dd=torch.stack([x.grad for x in dl]), dprop=pr.grad,
                dh0=hh.grad if hh.grad is not None else zero, dcoef=cf.grad)


def teacher_forced_out(ins, boundary, beta=0.75):
    """The read evaluated in fp64 on exactly what the kernel is given: the storage-dtype sources and the base as its
    caller forms it (the boundary blend is the caller's torch arithmetic in the storage dtype, looped_transformer.py:381)."""
    deltas, proposal, h0, q, prior, coeffs, up, up2 = ins
    base_st = proposal + beta * (h0 - proposal) if boundary else proposal
    _, cbar, c0 = TO.prologue(proposal.double(), h0.double(), coeffs.double(), prior.double(), beta, boundary)
    with torch.no_grad():
        out, tc = TO.read(base_st.double(), [x.double() for x in deltas], q.double(), cbar, c0, 1e-6, accumulate="exact")
    return out, tc


SHAPES32 = [(2, 64, 768), (2, 37, 1024), (1, 50, 1536), (1, 9, 3072), (1, 5, 64), (3, 7, 2048)]


@pytest.mark.parametrize("b,t,d", SHAPES32)
@pytest.mark.parametrize("n", [2, 3, 8, 16, 20])
@pytest.mark.parametrize("boundary", [False, True])
def test_read_fp32_all_gradients(FD, b, t, d, n, boundary):
    ins = cases.read_inputs(b, t, d, n, torch.float32, seed=1000 * n + d + int(boundary))
    got = run_read_gpu(FD, *ins, boundary)
    want = run_read_oracle(*ins, boundary, torch.float64, "exact")
    for k in want:
        if float(want[k].abs().max()) == 0.0:
            assert float(got[k].abs().max()) == 0.0, k
            continue
        assert rel(got[k], want[k]) < TOL32, (k, rel(got[k], want[k]))


@pytest.mark.parametrize("b,t,d", [(2, 256, 1024), (2, 128, 1536), (4, 128, 768), (1, 40, 3072)])
@pytest.mark.parametrize("n", [4, 16, 24])
def test_read_bf16_against_fp64(FD, b, t, d, n):
    """bf16 storage: the output within 2e-2 RMS of the fp32/fp64 evaluation of the same rounded inputs, and every
    gradient no worse than twice the reference's own bf16 error plus 2e-3 (tests/test_fused_dattn.py:96-108)."""
    ins = cases.read_inputs(b, t, d, n, torch.bfloat16, seed=7 * n + d)
    got = run_read_gpu(FD, *ins, True)
    ref_bf16 = run_read_oracle(*ins, True, torch.bfloat16, "storage")      # the reference's own arithmetic
    want = run_read_oracle(*ins, True, torch.float64, "exact")
    out_tf, _ = teacher_forced_out(ins, True)
    rms = float(out_tf.pow(2).mean().sqrt())
    err_out = float((got["out"].double().cpu() - out_tf).abs().max())
    assert err_out <= 2e-2 * rms, (err_out, rms)
    assert rel(got["tc"], want["tc"]) < 1e-4
    for k in want:
        if float(want[k].abs().max()) == 0.0:
            continue
        e_got, e_ref = rel(got[k], want[k]), rel(ref_bf16[k], want[k])
        assert e_got <= 2.0 * e_ref + 2e-3, (k, e_got, e_ref)


@pytest.mark.parametrize("b,t,d,n,dtype", [(1, 9, 4096, 5, torch.float32), (1, 9, 8192, 5, torch.bfloat16),
                                           (1, 11, 6144, 3, torch.bfloat16), (1, 40, 1024, 128, torch.float32),
                                           (1, 40, 1024, 128, torch.bfloat16), (2, 20, 2048, 96, torch.bfloat16)])
def test_read_at_the_limits(FD, b, t, d, n, dtype):
    """The widest rows the library takes (16 KiB: 32 chunks, sixteen warps per token in the backward) and the most
    sources (LB_MAX_SOURCES = 128: four passes of the scalar warps), forward and every gradient."""
    ins = cases.read_inputs(b, t, d, n, dtype, seed=3 * n + d)
    got = run_read_gpu(FD, *ins, True)
    want = run_read_oracle(*ins, True, torch.float64, "exact")
    if dtype == torch.float32:
        for k in want:
            if float(want[k].abs().max()) == 0.0:
                continue
            assert rel(got[k], want[k]) < 2e-5, (k, rel(got[k], want[k]))
        return
    ref_bf16 = run_read_oracle(*ins, True, torch.bfloat16, "storage")
    out_tf, _ = teacher_forced_out(ins, True)
    rms = float(out_tf.pow(2).mean().sqrt())
    assert float((got["out"].double().cpu() - out_tf).abs().max()) <= 2e-2 * rms
    assert rel(got["tc"], want["tc"]) < 1e-4
    for k in want:
        if float(want[k].abs().max()) == 0.0:
            continue
        e_got, e_ref = rel(got[k], want[k]), rel(ref_bf16[k], want[k])
        assert e_got <= 2.0 * e_ref + 2e-3, (k, e_got, e_ref)


@pytest.mark.parametrize("b,t,d,n,dtype", [(1, 64, 2048, 11, torch.bfloat16), (2, 100, 1024, 7, torch.float32),
                                           (1, 24, 512, 21, torch.bfloat16)])
def test_sources_per_stage_do_not_change_a_bit(FD, L, b, t, d, n, dtype):
    """Small tiles take 1, 2 or 4 sources per TMA stage; the order of the arithmetic does not depend on it."""
    ins = cases.read_inputs(b, t, d, n, dtype, seed=7 * n + d)
    got = []
    for sps in (1, 2, 4):
        L.set_option("fwd_sps", sps)
        got.append(run_read_gpu(FD, *ins, False))
    L.set_option("fwd_sps", 0)
    for other in got[1:]:
        for key in ("out", "tc", "dd", "dq"):
            assert torch.equal(got[0][key], other[key]), key


@pytest.mark.parametrize("b,t,d,n,dtype", [(1, 40, 1536, 11, torch.bfloat16), (1, 24, 3072, 9, torch.bfloat16),
                                           (1, 33, 2048, 6, torch.bfloat16), (1, 20, 1024, 7, torch.float32),
                                           (2, 50, 1024, 10, torch.bfloat16)])
def test_ring_depth_does_not_change_a_bit_in_the_backward(FD, L, b, t, d, n, dtype):
    """Rows split over several warps per token take their sources in groups of up to four, at most half the TMA ring
    at a time: with a ring of 2, 3, 5 or 8 stages the groups are 1, 1, 2 and 4 sources, and every sum is still formed in
    the same order (the one-warp-per-token shape in the list is there for the ring itself)."""
    ins = cases.read_inputs(b, t, d, n, dtype, seed=3 * n + d)
    got = []
    try:
        for stages in (0, 2, 3, 5, 8):
            L.set_option("bwd_stages", stages)
            got.append(run_read_gpu(FD, *ins, False))
    finally:
        L.reset_options()
    for other in got[1:]:
        for key in ("out", "tc", "dd", "dq", "dcoef"):
            assert torch.equal(got[0][key], other[key]), key
    assert L.device_error() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [2, 9, 16, 40])
def test_zero_query_identity_is_bitwise(FD, dtype, n):
    """Zero query and installed coefficients equal to the prior: out == base and tc == c0 bit for bit
    (tests/test_fused_dattn.py:109-125)."""
    b, t, d = 2, 40, 768
    deltas, proposal, h0, q, prior, coeffs, up, up2 = cases.read_inputs(b, t, d, n, dtype, seed=n, zero_query=True)
    coeffs = prior.view(1, 1, -1).expand(b, t, -1).contiguous()
    deltas = [x.cuda() for x in deltas]
    proposal, h0, prior, coeffs = proposal.cuda(), h0.cuda(), prior.cuda(), coeffs.cuda()
    for boundary in (False, True):
        base = proposal + 0.75 * (h0 - proposal) if boundary else proposal
        cbar = torch.cat((coeffs, torch.ones(b, t, 1, device="cuda")), -1)
        c0 = torch.cat((prior, torch.ones(1, device="cuda")), -1)
        if boundary:
            cbar, c0 = 0.25 * cbar, 0.25 * c0
        rstds = [FD.rstd(x, 1e-6) for x in deltas]
        with torch.no_grad():
            out, tc = FD.FusedDattnRead.apply(q.cuda(), base, cbar, c0, *deltas, *rstds)
        assert torch.equal(out, base)
        assert torch.equal(tc, c0.view(1, 1, -1).expand(b, t, -1))


# ------------------------------------------------------------------------------------------------------------
# 3. the fixtures generated by the unmodified reference
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("case", cases.READ_CASES, ids=[c[0] for c in cases.READ_CASES])
def test_golden_single_reads(FD, case):
    READS = np.load(os.path.join(G, "single_reads.npz"))
    name, b, t, d, n, dtn, seed, boundary = case
    ins = cases.read_inputs(b, t, d, n, DT[dtn], seed)
    assert cases.checksum(*ins[0], *ins[1:]) == pytest.approx(float(READS[f"{name}/checksum"]), rel=1e-12)
    got = run_read_gpu(FD, *ins, boundary)
    if dtn == "float32":
        for k in ("out", "tc", "dq", "dd", "dprop", "dh0", "dcoef"):
            want = READS[f"{name}/ref/{k}"]
            if np.abs(want).max() == 0:
                continue
            assert rel(got[k], want) < TOL32, (k, rel(got[k], want))
    else:
        # the reference's fp32 evaluation, moved onto the bf16 base the kernel is actually given (out = base + sum)
        proposal, h0 = ins[1], ins[2]
        base_bf16 = proposal + 0.75 * (h0 - proposal) if boundary else proposal
        base_f32 = proposal.float() + 0.75 * (h0.float() - proposal.float()) if boundary else proposal.float()
        want32 = READS[f"{name}/ref32/out"] + (base_bf16.float() - base_f32).numpy()
        rms = float(np.sqrt((want32.astype(np.float64) ** 2).mean()))
        assert float(np.abs(got["out"].float().cpu().numpy() - want32).max()) <= 2e-2 * rms
        assert rel(got["tc"], READS[f"{name}/ref32/tc"]) < 1e-4
        for k in ("dq", "dd", "dprop", "dh0", "dcoef"):
            w64 = READS[f"{name}/ref64/{k}"]
            if np.abs(w64).max() == 0:
                continue
            e_got, e_ref = rel(got[k], w64), rel(READS[f"{name}/ref/{k}"], w64)
            assert e_got <= 2.0 * e_ref + 2e-3, (k, e_got, e_ref)


def reference_combine(cell, FD, proposal, h0, deltas, coeffs, prior_coeffs, loop_idx, block_idx, keys=None, stack=None):
    """The stacked branch of the reference trainer cell's `combine`, restated on the test side
    (modeling_looped_transformer.py:148-169): the prologue in torch, then the exact call the trainer makes,
    FusedDattnReadStk.apply(stack, step, q, base, base_coeffs, next_prior, *deltas, *R_list)."""
    step = loop_idx * cell.num_blocks + block_idx
    at_boundary = block_idx == cell.num_blocks - 1
    base = proposal + cell.beta * (h0 - proposal) if at_boundary else proposal
    b, t, _ = proposal.shape
    one_tok = torch.ones(b, t, 1, device=proposal.device, dtype=torch.float32)
    one_prior = torch.ones(1, device=proposal.device, dtype=torch.float32)
    base_coeffs = one_tok if coeffs is None else torch.cat((coeffs, one_tok), dim=-1)
    next_prior = one_prior if prior_coeffs is None else torch.cat((prior_coeffs, one_prior), dim=-1)
    if at_boundary:
        r = 1.0 - cell.beta
        base_coeffs, next_prior = r * base_coeffs, r * next_prior
    if keys is not None and len(keys) < len(deltas):
        keys.append(stack.rstd(step, deltas[-1], cell.eps))
    if len(deltas) == 1:
        return base, base_coeffs, next_prior
    R_list = keys if keys is not None else [FD._alias(stack.R, i) for i in range(len(deltas))]
    out, target = FD.FusedDattnReadStk.apply(stack, step, cell.query[step - 1], base, base_coeffs, next_prior,
                                             *deltas, *R_list)
    return out, target, next_prior


# how the chain calls the read: the cell's fast path (prologue inside the kernels, one autograd node per step:
# FusedStepStk, no gradient stack: lb_step_bwd_deferred), the same with the gradient stack accumulated in place
# (lb_step_bwd), the same without the step node (FusedCombineStk), the cell with its prologue in torch
# (FusedDattnReadStk, the entry point the reference trainer calls), the reference's own combine restated above
COMBINE_PATHS = ["fused", "fused_rmw", "fused_combine", "dropin", "reference_combine"]


def chain_gpu(FD, h0, D, Q, Gu, K, R, beta, eps, scores, with_grad, list_layout=False, path="fused", use_keys=True):
    """The cell driven as the model drives it (blocks x -> x + D_s), on the GPU, through the drop-in module."""
    from loopback_b200.cell import LoopDeltaAttnRes
    N = K * R
    b, t, d = h0.shape
    cell = LoopDeltaAttnRes(d, R, K, beta=beta, eps=eps).cuda()
    cell.fuse_prologue = path in ("fused", "fused_rmw", "fused_combine")
    cell.fuse_step = path in ("fused", "fused_rmw")
    cell.deferred_grads = path == "fused"
    with torch.no_grad():
        if N > 1:
            cell.query.copy_(Q[:N - 1].cuda())
    h0g = h0.detach().clone().cuda().requires_grad_(with_grad)
    Dg = D.detach().clone().cuda().requires_grad_(with_grad)
    stack = None if list_layout else cell.new_stack((b, t, d), h0.dtype, "cuda", scores=scores)
    x, deltas, keys, coeffs, prior, states = h0g, [], ([] if use_keys else None), None, None, []
    with torch.set_grad_enabled(with_grad):
        loss = 0.0
        for s in range(N):
            l, blk = divmod(s, K)
            hs = x + Dg[s]
            deltas.append(stack.write(s, hs, x) if stack is not None else hs - x)
            if path == "reference_combine" and stack is not None:
                x, coeffs, prior = reference_combine(cell, FD, hs, h0g, deltas, coeffs, prior, l, blk, keys=keys, stack=stack)
            else:
                x, coeffs, prior = cell.combine(hs, h0g, deltas, coeffs, prior, l, blk, keys=keys, stack=stack)
            states.append(x)
            if with_grad:
                loss = loss + (x.float() * Gu[s].cuda()).sum()
        if with_grad:
            loss.backward()
    res = dict(states=torch.stack([s.detach() for s in states]), tc_last=coeffs.detach(), c0_last=prior.detach())
    if with_grad:
        res.update(dq=cell.query.grad.detach(), dD=Dg.grad.detach(), dh0=h0g.grad.detach())
    return res


@pytest.mark.parametrize("case", cases.CHAIN_CASES, ids=[c[0] for c in cases.CHAIN_CASES])
@pytest.mark.parametrize("path", ["scores", "stack", "list"])
@pytest.mark.parametrize("combine", COMBINE_PATHS)
def test_golden_chains(FD, case, path, combine):
    """K x R chains against the reference's states, tracked coefficients and gradients; `scores` is the stacked
    layout with cached scores (the trainer's default), `stack` the stacked layout without, `list` one tensor per
    update (tests/test_dattn_stack.py:96-118)."""
    CH = np.load(os.path.join(G, "small_chains.npz"))
    name, b, t, d, K, R, dtn, seed, with_grad = case
    h0, D, Q, Gu = cases.chain_inputs(b, t, d, K, R, seed, dtype=DT[dtn], sigma_q=0.3)
    assert cases.checksum(h0, D, Q, Gu) == pytest.approx(float(CH[f"{name}/checksum"]), rel=1e-12)
    N = K * R
    if path == "list" and combine != "fused":
        pytest.skip("the list layout has one combine path")
    got = chain_gpu(FD, h0, D, Q, Gu, K, R, 0.75, 1e-6, scores=path == "scores", with_grad=with_grad,
                    list_layout=path == "list", path=combine)
    assert torch.equal(got["c0_last"].cpu(), torch.from_numpy(CH[f"{name}/ref/c0_last"]))
    if dtn == "float32":
        assert rel(got["states"], CH[f"{name}/ref/states"]) < TOL32
        assert rel(got["tc_last"], CH[f"{name}/ref/tc_last"]) < TOL32
        if with_grad:
            assert rel(got["dq"], CH[f"{name}/ref/dq"]) < 3e-5
            assert rel(got["dD"], CH[f"{name}/ref/dD"]) < 3e-5
            assert rel(got["dh0"], CH[f"{name}/ref/dh0"]) < 3e-5
    else:
        # a chain compounds the bf16 state error of both implementations: norm-relative 3e-2 as the reference's
        # own stacked-layout test uses (tests/test_dattn_stack.py:108)
        def nrel(a, b_):
            a, b_ = a.double().cpu(), torch.from_numpy(np.asarray(b_, np.float64))
            return float((a - b_).norm() / b_.norm())
        assert nrel(got["states"], CH[f"{name}/ref32/states"]) < 3e-2
        assert nrel(got["dD"], CH[f"{name}/ref32/dD"]) < 3e-2
        assert nrel(got["dq"], CH[f"{name}/ref32/dq"]) < 3e-2
        assert nrel(got["dh0"], CH[f"{name}/ref32/dh0"]) < 3e-2


@pytest.mark.parametrize("combine", COMBINE_PATHS)
def test_config1_full_size(FD, combine):
    """benchmark configuration 1 (fp32, 512 tokens, d=768, K=4, R=4, seed 0): every read state against the
    reference's, at the stored tokens and through per-token sums of every state."""
    CFG1 = np.load(os.path.join(G, "cfg1_chain_fp32.npz"))
    c = cases.CFG1
    h0, D, Q, Gu = cases.chain_inputs(**c)
    assert cases.checksum(h0, D, Q, Gu) == pytest.approx(float(CFG1["checksum"]), rel=1e-12)
    N, n_tok, d = c["K"] * c["R"], c["b"] * c["t"], c["d"]
    for scores in (True, False):
        got = chain_gpu(FD, h0, D, Q, Gu, c["K"], c["R"], c["beta"], c["eps"], scores=scores, with_grad=False,
                        path=combine)
        st = got["states"].reshape(N, n_tok, d).cpu()
        tok = torch.from_numpy(CFG1["tokens"])
        assert rel(st[:, tok, :], CFG1["states_at_tokens"]) < TOL32
        assert rel(st.double().sum(dim=2), CFG1["token_sum"]) < TOL32
        assert rel(got["tc_last"].reshape(n_tok, N), CFG1["tc_last"]) < TOL32
        assert torch.equal(got["c0_last"].cpu(), torch.from_numpy(CFG1["c0_last"]))


# ------------------------------------------------------------------------------------------------------------
# 4. chains against the oracle at sizes the fixtures do not hold; teacher-forced bf16 protocol
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("write_kernel", [0, 3])      # by size / the tensor-core write where it applies
@pytest.mark.parametrize("d,K,R,n_tok", [(1024, 4, 6, 96), (1536, 6, 4, 40), (3072, 8, 3, 24), (2048, 5, 4, 64),
                                         (2048, 5, 16, 64)])
@pytest.mark.parametrize("combine", COMBINE_PATHS)
def test_bf16_chain_teacher_forced(FD, L, d, K, R, n_tok, write_kernel, combine):
    """Each read of a bf16 chain, given the GPU chain's own stored updates, base and installed coefficients,
    against the C oracle's fp32 evaluation of exactly those inputs: <= 2e-2 * RMS(out) max-abs per read."""
    from loopback_b200.cell import LoopDeltaAttnRes
    N = K * R
    L.set_option("write_tt", write_kernel)
    h0, D, Q, Gu = cases.chain_inputs(1, n_tok, d, K, R, seed=d + K, dtype=torch.bfloat16, sigma_d=0.3)
    cell = LoopDeltaAttnRes(d, R, K, beta=0.75, eps=1e-6).cuda()
    cell.fuse_prologue = combine in ("fused", "fused_rmw", "fused_combine")
    cell.fuse_step = combine in ("fused", "fused_rmw")
    with torch.no_grad():
        cell.query.copy_(Q[:N - 1].cuda())
    stack = cell.new_stack((1, n_tok, d), torch.bfloat16, "cuda", scores=True)
    h0g = h0.cuda()
    x, deltas, keys, coeffs, prior = h0g, [], [], None, None
    worst = 0.0
    with torch.no_grad():
        for s in range(N):
            l, blk = divmod(s, K)
            hs = x + D[s].cuda()
            deltas.append(stack.write(s, hs, x))
            cb_in, pr_in = coeffs, prior
            if combine == "reference_combine":
                x_new, coeffs, prior = reference_combine(cell, FD, hs, h0g, deltas, coeffs, prior, l, blk, keys=keys,
                                                         stack=stack)
            else:
                x_new, coeffs, prior = cell.combine(hs, h0g, deltas, coeffs, prior, l, blk, keys=keys, stack=stack)
            if s >= 1:
                base, cbar, c0 = TO.prologue(hs, h0g, cb_in, pr_in, 0.75, blk == K - 1)
                V = stack.V[:s + 1].float().cpu().numpy().reshape(s + 1, n_tok, d)
                Rr = stack.R[:s + 1].cpu().numpy().reshape(s + 1, n_tok)
                out, tc = CO.read_fwd(V, Rr, Q[s - 1].numpy(), base.float().cpu().numpy().reshape(n_tok, d),
                                      cbar.cpu().numpy().reshape(n_tok, s + 1), c0.cpu().numpy())
                rms = float(np.sqrt((out.astype(np.float64) ** 2).mean()))
                err = float(np.abs(x_new.float().cpu().numpy().reshape(n_tok, d) - out).max())
                worst = max(worst, err / rms)
                assert err <= 2e-2 * rms, (s, err, rms)
                assert rel(coeffs.reshape(n_tok, s + 1), tc) < 1e-4
            x = x_new
    L.set_option("write_tt", 0)
    print(f"d={d} N={N}: worst per-read error {worst:.3e} RMS")


@pytest.mark.parametrize("d,K,R,n_tok,dtype", [(768, 4, 4, 50, torch.float32), (1024, 4, 6, 33, torch.float32),
                                               (3072, 2, 3, 11, torch.float32), (64, 5, 16, 3, torch.float32)])
@pytest.mark.parametrize("scores", [True, False])
@pytest.mark.parametrize("combine", COMBINE_PATHS)
def test_fp32_chain_with_gradients(FD, d, K, R, n_tok, dtype, scores, combine):
    """fp32 chains, forward and the gradients of h0, every update and every query, against the C oracle (fp64)."""
    N = K * R
    h0, D, Q, Gu = cases.chain_inputs(1, n_tok, d, K, R, seed=3 * d + N, dtype=dtype, sigma_q=0.1)
    got = chain_gpu(FD, h0, D, Q, Gu, K, R, 0.75, 1e-6, scores=scores, with_grad=True, path=combine)
    want = CO.chain(h0.double().numpy().reshape(n_tok, d), D.double().numpy().reshape(N, n_tok, d),
                    Q.double().numpy(), Gu.double().numpy().reshape(N, n_tok, d), K, R, 0.75, 1e-6, False)
    assert rel(got["states"].reshape(N, n_tok, d), want["states"]) < TOL32
    assert rel(got["tc_last"].reshape(n_tok, N), want["tc_last"]) < TOL32
    assert rel(got["dq"], want["dq"][:N - 1]) < 3e-5
    assert rel(got["dD"].reshape(N, n_tok, d), want["dD"]) < 3e-5
    assert rel(got["dh0"].reshape(n_tok, d), want["dh0"]) < 3e-5


def oracle_chain_grads(h0, D, Q, Gu, K, R, hi, accumulate, scale_grads=True, beta=0.75, eps=1e-6):
    """The K x R chain in torch on the CPU (blocks x -> x + D_s) with autograd's gradients of sum_s <state_s, G_s>.
    hi = float64 with accumulate "exact": the chain evaluated exactly on the given (already rounded) inputs;
    hi = bfloat16 with accumulate "storage": the reference's own bf16 arithmetic, forward and backward.
    scale_grads=False cuts the gradient through the key scales (a caller that keeps no `keys`)."""
    ct = torch.float64 if hi == torch.float64 else torch.float32
    h0r = h0.detach().to(hi).clone().requires_grad_()
    Dr = D.detach().to(hi).clone().requires_grad_()
    Qr = Q.detach().to(ct).clone().requires_grad_()
    N = K * R
    x, sources, scales, tc, c0, loss, states = h0r, [], [], None, None, 0.0, []
    for s in range(N):
        h = x + Dr[s]
        v = h - x
        sources.append(v)
        r = TO.key_scale(v, eps)
        scales.append(r if scale_grads else r.detach())
        base, cbar, c0 = TO.prologue(h, h0r, tc, c0, beta, s % K == K - 1)
        if s == 0:
            x, tc = base, cbar
        else:
            out, tc = TO.read(base, sources, Qr[s - 1], cbar, c0, eps, accumulate=accumulate, scales=scales)
            x = out.to(hi)
        states.append(x.detach())
        loss = loss + (x.to(ct) * Gu[s].to(ct)).sum()
    loss.backward()
    return dict(states=torch.stack(states), dq=Qr.grad, dD=Dr.grad, dh0=h0r.grad)


@pytest.mark.parametrize("write_kernel", [0, 3])
@pytest.mark.parametrize("d,K,R,n_tok", [(1024, 4, 6, 160), (1536, 6, 4, 96), (3072, 8, 3, 64), (2048, 5, 4, 64)])
@pytest.mark.parametrize("combine", COMBINE_PATHS)
def test_bf16_chain_with_gradients(FD, L, d, K, R, n_tok, write_kernel, combine):
    """bf16 chains at the benchmark's row widths, through the stack with cached scores: the gradients of every query,
    every update and h0 against the chain evaluated in fp64 on the same bf16-rounded inputs, no worse than twice the
    error of the reference's own bf16 arithmetic plus 2e-3 (tests/test_fused_dattn.py:96-108). Covers the
    accumulating backward with the in-kernel finalisation, one and several warps per token, and the bf16 rounding of
    the gradient-stack accumulation."""
    L.set_option("write_tt", write_kernel)
    h0, D, Q, Gu = cases.chain_inputs(1, n_tok, d, K, R, seed=5 * d + K, dtype=torch.bfloat16, sigma_d=0.3, sigma_q=0.05)
    got = chain_gpu(FD, h0, D, Q, Gu, K, R, 0.75, 1e-6, scores=True, with_grad=True, path=combine)
    L.set_option("write_tt", 0)
    want = oracle_chain_grads(h0, D, Q, Gu, K, R, torch.float64, "exact")
    ref = oracle_chain_grads(h0, D, Q, Gu, K, R, torch.bfloat16, "storage")
    N = K * R
    for k in ("dq", "dD", "dh0"):
        w = want[k][:N - 1] if k == "dq" else want[k]
        rf = ref[k][:N - 1] if k == "dq" else ref[k]
        e_got, e_ref = rel(got[k], w), rel(rf, w)
        assert e_got <= 2.0 * e_ref + 2e-3, (k, e_got, e_ref)
    assert torch.isfinite(got["states"].float()).all()


@pytest.mark.parametrize("combine", ["dropin", "reference_combine"])
@pytest.mark.parametrize("scores", [True, False])
def test_fp32_chain_without_keys(FD, combine, scores):
    """A caller that passes keys=None (the scales are then plain slices of the stack, without a gradient path):
    same states; the query and h0 gradients are those of the chain with the key scales held constant. (The
    updates themselves get no gradient then, in the reference as here: their one gradient is handed out by the
    scale's node, fused_dattn.py:711-722.)"""
    d, K, R, n_tok = 256, 3, 3, 21
    N = K * R
    h0, D, Q, Gu = cases.chain_inputs(1, n_tok, d, K, R, seed=77, dtype=torch.float32, sigma_q=0.1)
    got = chain_gpu(FD, h0, D, Q, Gu, K, R, 0.75, 1e-6, scores=scores, with_grad=True, path=combine, use_keys=False)
    want = oracle_chain_grads(h0, D, Q, Gu, K, R, torch.float64, "exact", scale_grads=False)
    assert rel(got["states"], want["states"]) < TOL32
    assert rel(got["dq"], want["dq"][:N - 1]) < 3e-5
    assert rel(got["dh0"], want["dh0"]) < 3e-5


# ------------------------------------------------------------------------------------------------------------
# 5. interface behaviour the reference's tests pin
# ------------------------------------------------------------------------------------------------------------
def test_kept_loss_holds_no_stack(FD):
    """After the backward, a kept loss (and so its graph) holds no stack (tests/test_dattn_stack.py:161-198)."""
    from loopback_b200.cell import LoopDeltaAttnRes
    K, R, n_tok, d = 2, 4, 8192, 256

    def once():
        torch.manual_seed(0)
        cell = LoopDeltaAttnRes(d, R, K).cuda()
        with torch.no_grad():
            cell.query.normal_(0, 0.5)
        Ws = [(torch.randn(d, d, device="cuda") * 0.03).requires_grad_() for _ in range(K * R)]
        h0 = (torch.randn(1, n_tok, d, device="cuda") * 0.5).bfloat16().requires_grad_()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        stack = cell.new_stack((1, n_tok, d), torch.bfloat16, "cuda")
        h, deltas, keys, coeffs, prior = h0, [], [], None, None
        for s in range(K * R):
            l, blk = divmod(s, K)
            hs = (h.float() @ Ws[s]).bfloat16() + h
            deltas.append(stack.write(s, hs, h))
            h, coeffs, prior = cell.combine(hs, h0, deltas, coeffs, prior, l, blk, keys=keys, stack=stack)
        loss = (h.float() ** 2).mean()
        loss.backward()
        stack_bytes = 2 * (stack.V.numel() * 2 + stack.R.numel() * 4)
        del stack, h, hs, deltas, keys, coeffs, prior
        for p in (*Ws, h0, cell.query):
            p.grad = None
        torch.cuda.synchronize()
        return torch.cuda.memory_allocated() - before, stack_bytes, loss

    once()
    held, stack_bytes, kept = once()
    assert held < 0.05 * stack_bytes, (held, stack_bytes)


def test_error_behaviour(FD):
    from loopback_b200.cell import LoopDeltaAttnRes
    cell = LoopDeltaAttnRes(64, 2, 2).cuda()
    x = torch.zeros(1, 4, 64, device="cuda")
    with pytest.raises(ValueError):
        cell.combine(x, x, [x], None, None, 0, 2)
    with pytest.raises(ValueError):
        cell.combine(x, x, [x], None, None, 2, 0)
    with pytest.raises(ValueError):
        cell.combine(x, x, [x, x], None, None, 0, 0)
    stack = cell.new_stack((1, 4, 64), torch.float32, "cuda")
    with pytest.raises(RuntimeError):
        stack.write(0, x.bfloat16(), x.bfloat16())
    with pytest.raises(RuntimeError):
        FD.rstd(torch.zeros(4, 64), 1e-6)
    with pytest.raises(RuntimeError):
        FD.DattnStack(4, (1, 4, 64), torch.float32, "cpu")
    with pytest.raises(RuntimeError):
        FD.DattnStack(4, (1, 4, 63), torch.bfloat16, "cuda")
    d1 = stack.write(0, x + 1, x)
    with pytest.raises(RuntimeError):          # base of another dtype
        FD.FusedDattnReadStk.apply(stack, 1, torch.zeros(64, device="cuda"), x.bfloat16(),
                                   torch.ones(1, 4, 2, device="cuda"), torch.ones(2, device="cuda"), d1, d1,
                                   FD._alias(stack.R, 0), FD._alias(stack.R, 0))
    assert not FD.fused_read_supported(x.cpu(), [x.cpu()], [torch.ones(1, 4, 1)], torch.ones(1, 4, 1))


def test_a_wait_that_runs_out_unwinds_and_reports(L):
    """The kernels' waits are bounded. With the limit set to about a millisecond and the test hook that makes the first
    CTA's producer leave out one tile copy, that CTA's consumers give up their wait: the kernel RETURNS (nothing traps,
    nothing spins on), the device error word names the wait, the other CTAs' tokens are written as usual, and the
    next launch is unaffected."""
    n_tok, d, N, n = 2000, 1024, 8, 6
    g = torch.Generator(device="cuda").manual_seed(5)
    V = (torch.randn(N, n_tok, d, device="cuda", generator=g) * 0.5).bfloat16()
    R = torch.rsqrt(V.float().pow(2).mean(-1) + 1e-6).contiguous()
    dots = torch.randn(N, n_tok, device="cuda", generator=g)
    base = torch.randn(n_tok, d, device="cuda", generator=g).bfloat16()
    c0 = (torch.rand(n, device="cuda", generator=g) * 0.9 + 0.1).contiguous()
    cbar = (c0.view(1, -1) + 0.2 * torch.randn(n_tok, n, device="cuda", generator=g)).contiguous()

    def run():
        out = torch.full_like(base, float("nan"))
        tc = torch.empty(n_tok, n, device="cuda")
        L.check(L.lib().lb_read_fwd(L.ptr(V), L.ptr(R), L.ptr(dots), 0, L.ptr(base), L.ptr(cbar), L.ptr(c0), L.ptr(out),
                                    L.ptr(tc), None, None, None, n_tok, d, N, n, L.LB_DTYPE_BF16, L.stream_ptr()), "fwd")
        torch.cuda.synchronize()
        return out

    good = run()
    assert L.device_error() == 0 and torch.isfinite(good.float()).all()
    L.set_option("wait_cycles", 2_000_000)
    L.set_option("test_skip_item", 3)
    try:
        bad = run()
    finally:
        L.reset_options()
    assert L.device_error(clear=True) == 1, "the consumers' wait for a tile (code 1) must be on record"
    assert torch.equal(bad[8:1184], good[8:1184]), "tokens of the other CTAs are written as usual"
    assert torch.isnan(bad[:8].float()).any(), "the CTA that gave up stores nothing for the tile it could not finish"
    again = run()
    assert L.device_error() == 0 and torch.equal(again, good)


# ------------------------------------------------------------------------------------------------------------
# 6. full-size properties (benchmark configuration 2 shapes: 32768 tokens, d=1024, bf16, N=24)
# ------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("d,K,R,b,t", [(1024, 4, 6, 8, 4096), (1536, 6, 4, 16, 4096), (3072, 8, 3, 4, 4096)],
                         ids=["cfg2", "cfg3", "cfg4_rows_16384_tokens"])
def test_full_size_properties(FD, d, K, R, b, t):
    """At configuration 2's and 3's sizes the oracle is too slow, so the checks are properties: (a) per-token independence --
    the chain on the first 8192 tokens alone (still a batch the tensor-core write takes, with other tile sizes in all
    three kernels) reproduces the slice of the full chain bit for bit; (b) the tracked
    coefficients of every token sum to the read's mass; (c) zero queries reduce the chain to the decay-only closed
    form h0 + sum_i lambda^(R - floor(i/K)) D_i (within the bf16 state rounding), and tc == c0 bitwise."""
    N = K * R
    g = torch.Generator(device="cuda").manual_seed(0)
    h0 = torch.randn(b, t, d, device="cuda", generator=g).bfloat16()
    D = (torch.randn(N, b, t, d, device="cuda", generator=g) * 0.3).bfloat16()
    Q = torch.randn(N - 1, d, device="cuda", generator=g) * 0.02
    Gu = torch.randn(2, b, t, d, device="cuda", generator=g)

    def run(h0_, D_, Q_, grad, lo=0):
        from loopback_b200.cell import LoopDeltaAttnRes
        cell = LoopDeltaAttnRes(d, R, K).cuda()
        with torch.no_grad():
            cell.query.copy_(Q_)
        bb = h0_.shape[0]
        stack = cell.new_stack((bb, t, d), torch.bfloat16, "cuda")
        h0r = h0_.clone().requires_grad_(grad)
        x, deltas, keys, coeffs, prior = h0r, [], [], None, None
        loss = 0.0
        with torch.set_grad_enabled(grad):
            for s in range(N):
                l, blk = divmod(s, K)
                hs = x + D_[s]
                deltas.append(stack.write(s, hs, x))
                x, coeffs, prior = cell.combine(hs, h0r, deltas, coeffs, prior, l, blk, keys=keys, stack=stack)
                if grad:
                    loss = loss + (x.float() * Gu[s % 2, lo:lo + bb]).sum()
            if grad:
                loss.backward()
        return x.detach(), coeffs.detach(), prior.detach(), (h0r.grad, cell.query.grad) if grad else None

    x_full, tc_full, c0, grads_full = run(h0, D, Q, True)
    x_part, tc_part, _, grads_part = run(h0[:2], D[:, :2], Q, True)
    assert torch.equal(x_full[:2], x_part) and torch.equal(tc_full[:2], tc_part)
    assert torch.equal(grads_full[0][:2], grads_part[0])
    assert torch.isfinite(grads_full[1]).all() and torch.isfinite(grads_full[0]).all()
    # (a') the query gradient is a sum over tokens: the slices' gradients add up to the full batch's (fp32 round-off of
    # a different summation order), and every slice's loop-input gradient is the full one's slice, bit for bit
    dq_sum = grads_part[1].double()
    for lo in range(2, b, 2):
        _, _, _, gp = run(h0[lo:lo + 2], D[:, lo:lo + 2], Q, True, lo)
        assert torch.equal(grads_full[0][lo:lo + 2], gp[0])
        dq_sum += gp[1].double()
    assert float((dq_sum - grads_full[1].double()).abs().max()) < 2e-5 * float(grads_full[1].abs().max())
    assert float((tc_full.sum(-1) - c0.sum()).abs().max()) < 1e-4 * float(c0.sum())
    x_zero, tc_zero, c0z, _ = run(h0, D, torch.zeros_like(Q), False)
    assert torch.equal(tc_zero, c0z.view(1, 1, -1).expand_as(tc_zero))
    lam = 0.25
    closed = h0.float()
    for i in range(N):
        closed = closed + (lam ** (R - i // K)) * D[i].float()
    rms = float(closed.pow(2).mean().sqrt())
    assert float((x_zero.float() - closed).abs().max()) < 0.1 * rms
    assert float((x_zero.float() - closed).pow(2).mean().sqrt()) < 2e-2 * rms
