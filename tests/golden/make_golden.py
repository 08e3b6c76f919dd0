"""Generate the golden fixtures of this directory by running the UNMODIFIED reference on seeded inputs.

Run where the reference tree is available (it is imported, never copied):

    LOOPBACK_REF=/path/to/reference python tests/golden/make_golden.py

Writes cfg1_chain_fp32.npz, single_reads.npz and small_chains.npz next to this script. The reference entry point
used is LoopDeltaAttnRes.combine of the reference's looped_transformer.py with the fused path off (its default),
i.e. the reference read; gradients are the reference's autograd gradients.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import cases  # noqa: E402

REF = os.environ.get("LOOPBACK_REF")
if not REF or not os.path.isfile(os.path.join(REF, "looped_transformer.py")):
    raise SystemExit("set LOOPBACK_REF to a checkout of the reference (the directory holding looped_transformer.py)")
sys.path.insert(0, REF)
os.environ["LOOP_DATTN_FUSED"] = "0"
import looped_transformer as M  # noqa: E402  (the reference)

torch.set_num_threads(max(1, os.cpu_count() or 1))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float64": torch.float64}


def npy(x):
    x = x.detach()
    return (x.float() if x.dtype == torch.bfloat16 else x).numpy().copy()


def run_read(d, n, deltas, proposal, h0, q, prior, coeffs, up, up2, boundary, beta=0.75, eps=1e-6):
    """The reference read on one set of inputs, with all its gradients (cf. tests/test_fused_dattn.py:48-73)."""
    deltas = [x.detach().clone().requires_grad_() for x in deltas]
    proposal = proposal.detach().clone().requires_grad_()
    h0 = h0.detach().clone().requires_grad_()
    cf = coeffs.detach().clone().requires_grad_()
    mod = M.LoopDeltaAttnRes(d, num_loops=2, num_blocks=n if boundary else n + 1, beta=beta, eps=eps)
    with torch.no_grad():
        mod.query[n - 2].copy_(q)
    out, tc, nxt = mod.combine(proposal, h0, deltas, cf, prior, 0, n - 1)
    ((out.float() * up).sum() + (tc * up2).sum()).backward()
    zero = torch.zeros_like(proposal)
    return dict(out=npy(out), tc=npy(tc), c0=npy(nxt), dq=npy(mod.query.grad[n - 2]),
                dd=np.stack([npy(x.grad) for x in deltas]), dprop=npy(proposal.grad),
                dh0=npy(h0.grad if h0.grad is not None else zero), dcoef=npy(cf.grad))


def single_reads():
    store = {}
    for name, b, t, d, n, dtn, seed, boundary in cases.READ_CASES:
        dtype = DT[dtn]
        deltas, proposal, h0, q, prior, coeffs, up, up2 = cases.read_inputs(b, t, d, n, dtype, seed)
        store[f"{name}/checksum"] = np.float64(cases.checksum(*deltas, proposal, h0, q, prior, coeffs, up, up2))
        res = run_read(d, n, deltas, proposal, h0, q, prior, coeffs, up, up2, boundary)
        for k, v in res.items():
            store[f"{name}/ref/{k}"] = v
        # the same (rounded) inputs evaluated by the reference in fp64 -- and, for bf16 storage, in fp32
        for tag, hi in (("ref64", torch.float64),) + ((("ref32", torch.float32),) if dtype == torch.bfloat16 else ()):
            r = run_read(d, n, [x.to(hi) for x in deltas], proposal.to(hi), h0.to(hi), q.to(hi), prior.to(hi),
                         coeffs.to(hi), up.to(hi), up2.to(hi), boundary)
            for k, v in r.items():
                store[f"{name}/{tag}/{k}"] = v
    np.savez_compressed(os.path.join(HERE, "single_reads.npz"), **store)
    print("single_reads.npz:", len(cases.READ_CASES), "cases")


def run_chain(h0, D, Q, G, K, R, beta, eps, with_grad):
    """The reference cell driven as the model drives it (looped_transformer.py:513-546) with blocks x -> x + D_s."""
    N = K * R
    cell = M.LoopDeltaAttnRes(h0.shape[-1], R, K, beta=beta, eps=eps)
    with torch.no_grad():
        if N > 1:
            cell.query.copy_(Q[:N - 1])
    h0 = h0.detach().clone().requires_grad_(with_grad)
    D = D.detach().clone().requires_grad_(with_grad)
    x, deltas, keys, coeffs, prior, states = h0, [], [], None, None, []
    with torch.set_grad_enabled(with_grad):
        loss = 0.0
        for s in range(N):
            l, blk = divmod(s, K)
            hs = x + D[s]
            deltas.append(hs - x)
            x, coeffs, prior = cell.combine(hs, h0, deltas, coeffs, prior, l, blk, keys=keys)
            states.append(x)
            if with_grad:
                loss = loss + (x.float() * G[s]).sum()
        if with_grad:
            loss.backward()
    res = dict(states=np.stack([npy(s) for s in states]), tc_last=npy(coeffs), c0_last=npy(prior))
    if with_grad:
        res.update(dq=npy(cell.query.grad), dD=npy(D.grad), dh0=npy(h0.grad))
    return res


def small_chains():
    store = {}
    for name, b, t, d, K, R, dtn, seed, with_grad in cases.CHAIN_CASES:
        dtype = DT[dtn]
        h0, D, Q, G = cases.chain_inputs(b, t, d, K, R, seed, dtype=dtype, sigma_q=0.3)
        store[f"{name}/checksum"] = np.float64(cases.checksum(h0, D, Q, G))
        for k, v in run_chain(h0, D, Q, G, K, R, 0.75, 1e-6, with_grad).items():
            store[f"{name}/ref/{k}"] = v
        if dtype == torch.bfloat16:   # the same rounded inputs through the reference in fp32
            for k, v in run_chain(h0.float(), D.float(), Q, G, K, R, 0.75, 1e-6, with_grad).items():
                store[f"{name}/ref32/{k}"] = v
    np.savez_compressed(os.path.join(HERE, "small_chains.npz"), **store)
    print("small_chains.npz:", len(cases.CHAIN_CASES), "cases")


def cfg1():
    c = cases.CFG1
    h0, D, Q, G = cases.chain_inputs(**c)
    res = run_chain(h0, D, Q, G, c["K"], c["R"], c["beta"], c["eps"], with_grad=False)
    states = res["states"].reshape(c["K"] * c["R"], c["b"] * c["t"], c["d"])
    tok = np.array(cases.CFG1_TOKENS)
    store = dict(checksum=np.float64(cases.checksum(h0, D, Q, G)),
                 tokens=tok, states_at_tokens=states[:, tok, :].copy(),
                 state_sum=states.astype(np.float64).sum(axis=(1, 2)),
                 state_sumsq=(states.astype(np.float64) ** 2).sum(axis=(1, 2)),
                 state_absmax=np.abs(states).max(axis=(1, 2)),
                 token_sum=states.astype(np.float64).sum(axis=2),          # [N, n_tok]: every token of every state
                 tc_last=res["tc_last"].reshape(c["b"] * c["t"], -1), c0_last=res["c0_last"])
    np.savez_compressed(os.path.join(HERE, "cfg1_chain_fp32.npz"), **store)
    print("cfg1_chain_fp32.npz: states", states.shape, "stored tokens", len(tok))


if __name__ == "__main__":
    print("reference:", M.__file__)
    single_reads()
    small_chains()
    cfg1()
