"""The Loopback read cell on top of the CUDA kernels: a host-side mirror of the reference's `LoopDeltaAttnRes`.

Same constructor, parameter (`query`, (K R - 1, d), zero-initialised) and `combine` contract as the reference cell
(looped_transformer.py:334-424; the trainer model's copy adds the `stack=` argument), so a model loop written for the
reference runs unchanged.  Unlike the reference there is one path only -- the fused kernels -- and no environment
switch: inputs the kernels cannot take raise instead of silently taking an eager read.

    h_{s+1} = h_0 + sum_{i<=s} c_{s,i} d_i,    c_{s,i} = B_s softmax_i(q_s . rmsnorm(d_i) / sqrt(d) + log c0_{s,i})
    c0_{s,i} = lambda^(floor((s+1)/K) - floor(i/K)),   B_s = sum_i c0_{s,i},   lambda = 1 - beta
"""
from __future__ import annotations

import numpy as np
import torch
from torch import nn

from . import fused_dattn as FD


class LoopDeltaAttnRes(nn.Module):
    def __init__(self, hidden_size: int, num_loops: int, num_blocks: int, beta: float = 0.75, eps: float = 1e-6):
        super().__init__()
        if num_loops < 1 or num_blocks < 1:
            raise ValueError(f"delta_attnres needs positive num_loops/num_blocks, got {num_loops}/{num_blocks}")
        if not 0.0 <= float(beta) < 1.0:
            raise ValueError(f"delta_attnres needs 0 <= beta < 1, got {beta}")
        self.dim = int(hidden_size)
        self.num_loops = int(num_loops)
        self.num_blocks = int(num_blocks)
        self.num_steps = self.num_loops * self.num_blocks
        self.beta = float(beta)
        self.eps = float(eps)
        self.query = nn.Parameter(torch.zeros(self.num_steps - 1, self.dim))
        self.fuse_prologue = True      # fold the boundary blend and the coefficient append/decay into the kernels
        self.fuse_step = True          # ... and make the write and the read of a step one autograd node
        self.deferred_grads = True     # ... whose backward keeps no gradient stack (DattnStack.deferred_grads)
        self.__dict__["peer_reduce"] = None   # see enable_peer_reduce (not a submodule, not part of the state dict)
        self.reset_parameters()

    def enable_peer_reduce(self, device, group=None):
        """Data parallel over the GPUs of one NVLink node: from now on the pass's last backward sums the query gradient
        over the ranks of `group` itself, through peer memory (dist.PeerQueryGrad), and `query.grad` arrives summed;
        the caller (or its data-parallel wrapper) must not reduce it again. Collective: every rank calls it once."""
        from .dist import PeerQueryGrad
        self.__dict__["peer_reduce"] = PeerQueryGrad((self.num_steps - 1, self.dim), device, group)
        return self.peer_reduce

    def reset_parameters(self):
        with torch.no_grad():
            self.query.zero_()

    def prior_rows(self, device) -> torch.Tensor:
        """[N, N] fp32 on `device`: row s holds, in its first s + 1 entries, the prior of read s -- built on the host
        exactly as the reads build it step by step (append 1; multiply everything by 1 - beta when an iteration
        ends, in fp32), so a pass needs no per-read cat / multiply kernels for it."""
        key = str(torch.device(device))
        cache = self.__dict__.setdefault("_prior_cache", {})
        if key not in cache:
            N = self.num_steps
            table = np.zeros((N, N), np.float32)
            c = np.zeros(0, np.float32)
            for s in range(N):
                c = np.concatenate((c, np.ones(1, np.float32)))
                if s % self.num_blocks == self.num_blocks - 1:
                    c = (np.float32(1.0 - self.beta) * c).astype(np.float32)
                table[s, :s + 1] = c
            rows = torch.from_numpy(table).to(device)
            # per read: the prior row's address (how combine recognises a prior it handed out) and the row itself
            cache[key] = (rows, float(self.beta), [rows[s].data_ptr() for s in range(N)],
                          [rows[s, :s + 1] for s in range(N)])
        if cache[key][1] != float(self.beta):
            del cache[key]
            return self.prior_rows(device)
        return cache[key][0]

    def _prior_views(self, device):
        self.prior_rows(device)
        entry = self.__dict__["_prior_cache"][str(torch.device(device))]
        return entry[2], entry[3]

    def new_stack(self, shape, dtype, device, scores: bool = True, fuse_decode: bool = True) -> FD.DattnStack:
        """The per-forward storage the model creates before its loop over the shared blocks (the trainer model's
        forward does this inline); `scores` caches each update's scores at its write (LOOP_DATTN_DOTS).
        `fuse_decode`: for decode-sized batches without autograd, a write is launched together with the read that
        follows it, as one kernel (see DattnStack.defer_writes)."""
        stack = FD.DattnStack(self.num_steps, tuple(shape), dtype, device, query=self.query if scores else None,
                              eps=self.eps)
        stack.defer_writes = bool(fuse_decode and scores)
        stack.deferred_grads = bool(self.deferred_grads)
        stack.peer_reduce = self.peer_reduce
        return stack

    def combine(self, proposal, h0, deltas, coeffs, prior_coeffs, loop_idx, block_idx, keys=None, stack=None):
        """One read after application `block_idx` of iteration `loop_idx`.

        proposal  the block output (b, t, d);  h0 the loop input;  deltas the updates stored so far (this one last);
        coeffs    the coefficients the previous read installed, (b, t, n - 1) fp32, None at the first read;
        prior_coeffs  the previous read's prior (n - 1,) fp32, None at the first read;
        keys      optional caller-owned cache of the updates' key scales, extended here by one;
        stack     the pass's DattnStack when the updates are its slices (the fast path).
        Returns (next state, installed coefficients, this read's prior)."""
        if not 0 <= block_idx < self.num_blocks:
            raise ValueError(f"delta_attnres block_idx={block_idx}, need [0,{self.num_blocks})")
        step = loop_idx * self.num_blocks + block_idx
        if step >= self.num_steps:
            raise ValueError(f"delta_attnres step {step} exceeds constructed depth {self.num_steps}")
        if len(deltas) != step + 1:
            raise ValueError(f"delta_attnres step {step} received {len(deltas)} deltas, expected {step + 1}")

        closes_iteration = block_idx == self.num_blocks - 1
        if self.fuse_prologue and stack is not None and step >= 1 and coeffs is not None and proposal.is_contiguous() \
                and (not closes_iteration or h0.is_contiguous()):
            row_ptrs, row_views = self._prior_views(proposal.device)
            if prior_coeffs is not None and prior_coeffs.data_ptr() == row_ptrs[step - 1]:
                # the whole prologue (boundary blend, appended 1, decay) runs inside the kernels
                lam = 1.0 - self.beta if closes_iteration else 1.0
                c0 = row_views[step]
                pend = stack._pending
                if (pend is not None and pend[0] == step and pend[1] is proposal and coeffs.dtype == torch.float32
                        and coeffs.is_contiguous() and not torch.is_grad_enabled()):
                    # decode-sized batch, no autograd: the recorded write and this read are one launch
                    if keys is not None and len(keys) < len(deltas):
                        keys.append(stack.R[step])
                    out, tc = stack.step_forward(step, proposal, pend[2], h0 if closes_iteration else None, self.beta,
                                                 coeffs, lam, c0)
                    return out, tc.view(*proposal.shape[:-1], step + 1), c0
                w = stack._last_write
                if (self.fuse_step and keys is not None and w is not None and w[0] == step and w[1] is proposal
                        and len(keys) >= step and (step > 1 or len(keys) >= 1)):
                    # one autograd node for the step: the write's tensors come from the stack, no update or scale is
                    # an input (step 1 excepted, which finishes update 0)
                    stack._last_write = None
                    if len(keys) < len(deltas):
                        keys.append(FD._alias(stack.R, step))
                    first = (deltas[0], keys[0]) if step == 1 else ()
                    out, tc = FD.FusedStepStk.apply(stack, step, self.query, proposal, w[2],
                                                    h0 if closes_iteration else None, self.beta, coeffs, lam, c0, *first)
                    return out, tc, c0
                if keys is not None and len(keys) < len(deltas):
                    keys.append(stack.rstd(step, deltas[-1], self.eps))
                scales = keys if keys is not None else [FD._alias(stack.R, i) for i in range(len(deltas))]
                out, tc = FD.FusedCombineStk.apply(stack, step, self.query[step - 1], proposal,
                                                   h0 if closes_iteration else None, self.beta, coeffs, lam, c0,
                                                   *deltas, *scales)
                return out, tc, c0
        base = proposal + self.beta * (h0 - proposal) if closes_iteration else proposal
        ones_tok = torch.ones(*proposal.shape[:-1], 1, device=proposal.device, dtype=torch.float32)
        ones_one = torch.ones(1, device=proposal.device, dtype=torch.float32)
        cbar = ones_tok if coeffs is None else torch.cat((coeffs, ones_tok), dim=-1)
        c0 = ones_one if prior_coeffs is None else torch.cat((prior_coeffs, ones_one), dim=-1)
        if closes_iteration:
            lam = 1.0 - self.beta
            cbar, c0 = lam * cbar, lam * c0

        if stack is not None:
            if keys is not None and len(keys) < len(deltas):
                keys.append(stack.rstd(step, deltas[-1], self.eps))
            if step == 0:
                if prior_coeffs is None:
                    c0 = self.prior_rows(proposal.device)[0, :1]      # same values; lets the next reads fuse
                return base, cbar, c0
            scales = keys if keys is not None else [FD._alias(stack.R, i) for i in range(len(deltas))]
            out, tc = FD.FusedDattnReadStk.apply(stack, step, self.query[step - 1], base.contiguous(), cbar, c0,
                                                 *deltas, *scales)
            return out, tc, c0

        if keys is not None and len(keys) < len(deltas):
            keys.append(FD.rstd(deltas[-1], self.eps))
        if step == 0:
            return base, cbar, c0
        scales = keys if keys is not None else [FD.rstd(v, self.eps) for v in deltas]
        if not FD.fused_read_supported(base, deltas, scales, cbar):
            raise RuntimeError("delta_attnres: the fused read does not support this layout "
                               "(CUDA, contiguous, one dtype in {bf16, fp32}, row size a multiple of 16 bytes)")
        out, tc = FD.FusedDattnRead.apply(self.query[step - 1], base, cbar, c0, *deltas, *scales)
        return out, tc, c0


def install(reference_model_module, fused_module=FD) -> None:
    """Make a reference model module (the port `looped_transformer` or the trainer's
    `modeling_looped_transformer`) use this package as its fused read: it sets the module-level cache its
    `_fused_dattn()` consults, exactly what the reference's own tests do to switch paths."""
    reference_model_module._FUSED_DATTN = fused_module
