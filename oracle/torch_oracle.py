"""Differentiable torch-CPU restatement of the Loopback read. TEST INFRASTRUCTURE, NOT PRODUCT.

A functional restatement (stacked sources, no module state) of what the reference cell computes; gradients come
from autograd, so this is the checker for every gradient the CUDA backward produces. Reference lines restated:
    key scale / key   looped_transformer.py:307-309, :406
    prologue          looped_transformer.py:380-391
    read body         looped_transformer.py:410-424   (first read: :407-408)
Pinned against the reference's own tensors in tests/golden/ (see make_golden.py there).
"""
from __future__ import annotations

import math

import torch


def key_scale(v: torch.Tensor, eps: float) -> torch.Tensor:
    """rsqrt(mean(v^2) + eps) over the last axis, keepdim; computed in fp32 for bf16 inputs (:406 casts first)."""
    vf = v.float() if v.dtype == torch.bfloat16 else v
    return torch.rsqrt(vf.square().mean(dim=-1, keepdim=True) + eps)


def decay_prior(step: int, num_blocks: int, beta: float, device="cpu") -> torch.Tensor:
    """The prior of read `step` ([step + 1], fp32), by append-and-decay (:385-391)."""
    c0 = torch.empty(0, dtype=torch.float32, device=device)
    one = torch.ones(1, dtype=torch.float32, device=device)
    for s in range(step + 1):
        c0 = torch.cat((c0, one))
        if s % num_blocks == num_blocks - 1:
            c0 = (1.0 - beta) * c0
    return c0


def prologue(proposal, h0, tc_prev, c0_prev, beta: float, at_boundary: bool):
    """(base, cbar, c0) entering a read (:380-391). tc_prev [..., n-1] or None; c0_prev [n-1] or None."""
    base = proposal + beta * (h0 - proposal) if at_boundary else proposal
    one_tok = torch.ones(*proposal.shape[:-1], 1, dtype=torch.float32, device=proposal.device)
    one = torch.ones(1, dtype=torch.float32, device=proposal.device)
    cbar = one_tok if tc_prev is None else torch.cat((tc_prev, one_tok), dim=-1)
    c0 = one if c0_prev is None else torch.cat((c0_prev, one), dim=-1)
    if at_boundary:
        cbar, c0 = (1.0 - beta) * cbar, (1.0 - beta) * c0
    return base, cbar, c0


def read(base, sources, q, cbar, c0, eps: float, accumulate: str = "exact", scales=None):
    """One read over `sources` (a list of n tensors [..., d]); returns (out, tc).

    accumulate = "exact":   coefficient deltas and the sum stay in the compute type of `q`/scores (fp32, or fp64
                            when everything is fp64) and nothing is rounded -- "the reference read evaluated in
                            fp32 on the same inputs";
               = "storage": the reference's own order -- deltas cast to the activation dtype, terms and the running
                            sum in that dtype (:419-424).
    `scales`, if given, are the sources' key scales (so a caller can route gradients through them separately).
    Scores are fp32 unless the sources are fp64, in which case they are fp64 (a true fp64 evaluation; the reference
    itself casts keys and query to fp32 even then, :406, :411)."""
    n = len(sources)
    act = base.dtype
    ct = torch.float64 if sources[0].dtype == torch.float64 else torch.float32
    d = sources[0].shape[-1]
    if scales is None:
        scales = [key_scale(v, eps) for v in sources]
    qf = q.to(ct)
    inv = 1.0 / math.sqrt(d)
    z = torch.stack([((v.to(ct) * r.to(ct)) * qf).sum(-1) for v, r in zip(sources, scales)], dim=-1) * inv
    lc = torch.log(c0.to(ct).clamp_min(1e-8))
    p0 = torch.softmax(lc, dim=-1)
    p = torch.softmax(z + lc, dim=-1)
    tc = c0.to(ct) + c0.to(ct).sum() * (p - p0)
    w = tc - cbar.to(ct)
    if accumulate == "storage":
        w = w.to(act)
        corr = None
        for i, v in enumerate(sources):
            term = w[..., i:i + 1] * v
            corr = term if corr is None else corr + term
        return base + corr, tc
    corr = None
    for i, v in enumerate(sources):
        term = w[..., i:i + 1] * v.to(ct)
        corr = term if corr is None else corr + term
    return base.to(ct) + corr, tc


def chain(h0, D, Q, num_blocks: int, num_loops: int, beta: float, eps: float, accumulate: str = "storage"):
    """A K x R pass with the blocks replaced by x -> x + D_s. Returns (states list, tc_last, c0_last).
    Model loop restated: looped_transformer.py:513-546."""
    N = num_blocks * num_loops
    x, sources, scales, tc, c0, states = h0, [], [], None, None, []
    for s in range(N):
        blk = s % num_blocks
        h = x + D[s]
        v = h - x
        sources.append(v)
        scales.append(key_scale(v, eps))
        base, cbar, c0 = prologue(h, h0, tc, c0, beta, blk == num_blocks - 1)
        if s == 0:
            x, tc = base, cbar
        else:
            out, tc = read(base, sources, Q[s - 1], cbar, c0, eps, accumulate=accumulate, scales=scales)
            x = out.to(h0.dtype) if accumulate == "storage" else out
        states.append(x)
    return states, tc, c0
