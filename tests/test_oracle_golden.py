"""The CPU oracle (both restatements) against tensors produced by the unmodified reference (tests/golden/)."""
import os

import numpy as np
import pytest
import torch

import cases
from oracle import c_oracle as CO
from oracle import torch_oracle as TO

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
READS = np.load(os.path.join(G, "single_reads.npz"))
CHAINS = np.load(os.path.join(G, "small_chains.npz"))
CFG1 = np.load(os.path.join(G, "cfg1_chain_fp32.npz"))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel(a, b):
    """max-abs error over max-abs reference, the measure of the reference's own kernel test (test_fused_dattn.py:76)."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def read_setup(case):
    name, b, t, d, n, dtn, seed, boundary = case
    ins = cases.read_inputs(b, t, d, n, DT[dtn], seed)
    assert cases.checksum(*ins[0], *ins[1:]) == pytest.approx(float(READS[f"{name}/checksum"]), rel=1e-12), \
        "seeded inputs changed: regenerate the fixtures where the reference is available"
    return ins


@pytest.mark.parametrize("case", cases.READ_CASES, ids=[c[0] for c in cases.READ_CASES])
def test_torch_oracle_single_read(case):
    """Forward and all seven gradients of one read, torch restatement vs the reference, same dtype."""
    name, b, t, d, n, dtn, seed, boundary = case
    deltas, proposal, h0, q, prior, coeffs, up, up2 = read_setup(case)
    for tag, hi in (("ref", DT[dtn]), ("ref64", torch.float64)):
        dl = [x.detach().to(hi).clone().requires_grad_() for x in deltas]
        pr, hh = (x.detach().to(hi).clone().requires_grad_() for x in (proposal, h0))
        cf = coeffs.detach().to(torch.float64 if hi == torch.float64 else torch.float32).clone().requires_grad_()
        qq = q.detach().to(hi if hi == torch.float64 else torch.float32).clone().requires_grad_()
        base, cbar, c0 = TO.prologue(pr, hh, cf, prior.to(cf.dtype), 0.75, boundary)
        out, tc = TO.read(base, dl, qq, cbar, c0, 1e-6, accumulate="storage")
        ((out.float() * up).sum() + (tc * up2).sum()).backward() if hi != torch.float64 else \
            ((out * up.double()).sum() + (tc * up2.double()).sum()).backward()
        got = dict(out=out, tc=tc, dq=qq.grad, dd=torch.stack([x.grad for x in dl]), dprop=pr.grad,
                   dh0=hh.grad if hh.grad is not None else torch.zeros_like(hh), dcoef=cf.grad)
        # fp32: summation order only; bf16: identical op sequence, so roundings coincide almost everywhere;
        # "ref64" has fp32 scores in the reference and fp64 scores here
        tol = 2e-6 if hi == torch.float32 else (2e-2 if hi == torch.bfloat16 else 2e-6)
        for k, v in got.items():
            want = READS[f"{name}/{tag}/{k}"]
            if np.abs(want).max() == 0:
                assert float(v.detach().abs().max()) == 0
                continue
            assert rel(v.detach().double().numpy(), want) < tol, (name, tag, k)


@pytest.mark.parametrize("case", cases.READ_CASES, ids=[c[0] for c in cases.READ_CASES])
def test_c_oracle_single_read(case):
    """C restatement: fp32 flavour vs the reference's fp32 run, fp64 flavour vs its fp64 run (analytic backward)."""
    name, b, t, d, n, dtn, seed, boundary = case
    deltas, proposal, h0, q, prior, coeffs, up, up2 = read_setup(case)
    bf16 = dtn == "bfloat16"
    for tag, nt in ((("ref32" if bf16 else "ref"), np.float32), ("ref64", np.float64)):
        V = np.stack([x.float().numpy().reshape(b * t, d) for x in deltas]).astype(nt)
        prop = proposal.float().numpy().reshape(b * t, d).astype(nt)
        hh = h0.float().numpy().reshape(b * t, d).astype(nt)
        base = CO.base_blend(prop, hh, 0.75, boundary, bf16_storage=False)
        lam = np.float32(0.25) if boundary else np.float32(1.0)
        c0 = (np.concatenate([prior.numpy(), np.ones(1, np.float32)]) * lam).astype(np.float32)
        cbar = (np.concatenate([coeffs.numpy().reshape(b * t, n - 1), np.ones((b * t, 1), np.float32)], 1)
                * lam).astype(nt)
        R = np.stack([CO.write(V[i], np.zeros_like(V[i]), 1e-6, False)[1] for i in range(n)])
        qn = q.numpy().astype(nt)
        out, tc = CO.read_fwd(V, R, qn, base, cbar, c0)
        g = up.numpy().reshape(b * t, d).astype(nt)
        gt = up2.numpy().reshape(b * t, n).astype(nt)
        dq, dV, dcbar = CO.read_bwd(V, R, qn, cbar, c0, g, gt)
        want = {k: READS[f"{name}/{tag}/{k}"] for k in ("out", "tc", "dq", "dd", "dprop", "dh0", "dcoef")}
        tol = 3e-6
        assert rel(out, want["out"].reshape(b * t, d)) < tol
        assert rel(tc, want["tc"].reshape(b * t, n)) < tol
        assert rel(dq, want["dq"]) < tol
        assert rel(dV, want["dd"].reshape(n, b * t, d)) < tol
        assert rel(dcbar[:, :n - 1] * lam, want["dcoef"].reshape(b * t, n - 1)) < tol
        dprop = g * (0.25 if boundary else 1.0)
        assert rel(dprop, want["dprop"].reshape(b * t, d)) < tol
        if boundary:
            assert rel(g * 0.75, want["dh0"].reshape(b * t, d)) < tol


@pytest.mark.parametrize("case", cases.CHAIN_CASES, ids=[c[0] for c in cases.CHAIN_CASES])
def test_oracles_small_chains(case):
    """K x R chains (blocks x -> x + D_s): every state, the tracked coefficients and all gradients."""
    name, b, t, d, K, R, dtn, seed, with_grad = case
    h0, D, Q, Gu = cases.chain_inputs(b, t, d, K, R, seed, dtype=DT[dtn], sigma_q=0.3)
    assert cases.checksum(h0, D, Q, Gu) == pytest.approx(float(CHAINS[f"{name}/checksum"]), rel=1e-12)
    N = K * R
    bf16 = dtn == "bfloat16"
    want = {k.split("/")[-1]: CHAINS[k] for k in CHAINS.files if k.startswith(f"{name}/ref/")}
    # torch restatement, reference accumulation order, same dtype
    hh, DD = h0.clone().requires_grad_(with_grad), D.clone().requires_grad_(with_grad)
    QQ = Q.clone().requires_grad_(with_grad)
    with torch.set_grad_enabled(with_grad):
        states, tc, c0 = TO.chain(hh, DD, QQ, K, R, 0.75, 1e-6, accumulate="storage")
        if with_grad:
            sum((s.float() * Gu[i]).sum() for i, s in enumerate(states)).backward()
    tol = 2e-2 if bf16 else 5e-6
    assert rel(torch.stack(states).detach().float().numpy(), want["states"]) < tol
    assert rel(tc.detach().numpy(), want["tc_last"]) < (1e-3 if bf16 else 5e-6)
    assert np.array_equal(c0.numpy(), want["c0_last"])
    if with_grad:
        assert rel(QQ.grad[:N - 1].numpy(), want["dq"]) < (5e-2 if bf16 else 2e-5)
        assert rel(DD.grad.float().numpy(), want["dD"]) < (5e-2 if bf16 else 2e-5)
        assert rel(hh.grad.float().numpy(), want["dh0"]) < (5e-2 if bf16 else 2e-5)
    # C restatement (fp32 flavour); for bf16 storage it reproduces the reference's bf16 accumulation order
    res = CO.chain(h0.float().numpy().reshape(b * t, d), D.float().numpy().reshape(N, b * t, d),
                   Q.numpy().astype(np.float32), Gu.numpy().reshape(N, b * t, d) if with_grad else None,
                   K, R, 0.75, 1e-6, bf16)
    assert rel(res["states"], want["states"].reshape(N, b * t, d)) < tol
    assert rel(res["tc_last"], want["tc_last"].reshape(b * t, N)) < (1e-3 if bf16 else 5e-6)
    if with_grad:
        # the C backward is exact-arithmetic fp32 (no bf16 rounding of gradients): compare with the reference's
        # fp32 evaluation of the same rounded inputs when storage is bf16
        tag = "ref32" if bf16 else "ref"
        if bf16:
            res = CO.chain(h0.float().numpy().reshape(b * t, d), D.float().numpy().reshape(N, b * t, d),
                           Q.numpy().astype(np.float32), Gu.numpy().reshape(N, b * t, d), K, R, 0.75, 1e-6, False)
            assert rel(res["states"], CHAINS[f"{name}/ref32/states"].reshape(N, b * t, d)) < 5e-6
        assert rel(res["dq"][:N - 1], CHAINS[f"{name}/{tag}/dq"]) < 2e-5
        assert rel(res["dD"], CHAINS[f"{name}/{tag}/dD"].reshape(N, b * t, d)) < 2e-5
        assert rel(res["dh0"], CHAINS[f"{name}/{tag}/dh0"].reshape(b * t, d)) < 2e-5


def test_clamped_prior_case_is_exercised():
    """The K=5, R=16 chain drives the prior below the reference's 1e-8 clamp, where tc != mass * p."""
    c0, lc, mass = CO.prior(79, 5, 0.75)
    assert c0.min() < 1e-8 and np.isclose(lc.min(), np.log(np.float32(1e-8)))
    assert np.array_equal(c0, CHAINS["f32_k5r16_clamp/ref/c0_last"])
    assert np.array_equal(c0, TO.decay_prior(79, 5, 0.75).numpy())


def test_config1_chain_fp32():
    """benchmark configuration 1 at full size through the C oracle (fp32) and the torch restatement."""
    c = cases.CFG1
    h0, D, Q, Gu = cases.chain_inputs(**c)
    assert cases.checksum(h0, D, Q, Gu) == pytest.approx(float(CFG1["checksum"]), rel=1e-12)
    N, n_tok, d = c["K"] * c["R"], c["b"] * c["t"], c["d"]
    res = CO.chain(h0.numpy().reshape(n_tok, d), D.numpy().reshape(N, n_tok, d), Q.numpy(), None,
                   c["K"], c["R"], c["beta"], c["eps"], False)
    states = res["states"]
    tok = CFG1["tokens"]
    assert rel(states[:, tok, :], CFG1["states_at_tokens"]) < 1e-5
    assert rel(states.astype(np.float64).sum(axis=2), CFG1["token_sum"]) < 1e-5
    assert rel(res["tc_last"], CFG1["tc_last"]) < 1e-5
    with torch.no_grad():
        st, tc, c0 = TO.chain(h0, D, Q, c["K"], c["R"], c["beta"], c["eps"])
    st = torch.stack(st).reshape(N, n_tok, d).numpy()
    assert rel(st[:, tok, :], CFG1["states_at_tokens"]) < 1e-5
    assert rel((st.astype(np.float64) ** 2).sum(axis=(1, 2)), CFG1["state_sumsq"]) < 1e-6
    assert np.array_equal(c0.numpy(), CFG1["c0_last"])
