"""Drop-in replacement of the reference's `fused_dattn` module, backed by the sm_100a CUDA kernels.

Same names, argument meaning and error behaviour as the reference module the models import lazily
(looped_transformer.py:315-331 and the trainer model's `_fused_dattn()`): `rstd`, `fused_read_supported`,
`FusedDattnRead`, `DattnStack` (+ `write`, `rstd`, `grads`), `_alias`, `FusedDattnReadStk`.  One read at step s has
n = s + 1 sources, the raw block updates v_i, and computes

    z_i  = r_i (q . v_i) / sqrt(d)                       r_i the key scale of v_i (an input with its own gradient)
    p    = softmax_i(z_i + lc_i),  p0 = softmax_i(lc_i)   lc_i = log max(c0_i, 1e-8),  M = sum_i c0_i
    tc_i = c0_i + M (p_i - p0_i)                          the installed coefficients, returned for the next read
    out  = base + sum_i (tc_i - cbar_i) v_i               cbar_i the coefficients installed by the previous read

exactly as the reference read (LoopDeltaAttnRes.combine, looped_transformer.py:405-424).  Differences from the
reference module are confined to private details: the score cache DOTS is laid out [query][update][token], only the
queries that will read an update are scored at its write, the log-prior and the mass are formed inside the kernels,
and the backward is one kernel.  There is no CPU or eager fallback: unsupported inputs raise.
"""
from __future__ import annotations

import torch

from . import _lib
from ._lib import check, dtype_code, ptr, stream_ptr

__all__ = ["rstd", "fused_read_supported", "FusedDattnRead", "DattnStack", "_alias", "FusedDattnReadStk",
           "FusedCombineStk", "FusedStepStk"]


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


_NO_GUARD = _NoGuard()


def _on(dev):
    """A device guard that costs nothing when `dev` is already the current device (the usual case)."""
    return _NO_GUARD if dev.index is None or dev.index == torch.cuda.current_device() else torch.cuda.device(dev)


def _require_cuda(t: torch.Tensor, what: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"loopback_b200.{what}: tensors must live on a CUDA device (there is no CPU path)")


# --------------------------------------------------------------------------------------------------------------
# the key scale of a free-standing update (list layout)            reference: fused_dattn.py:197-261
# --------------------------------------------------------------------------------------------------------------
class _Rstd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, eps: float):
        xc = x.contiguous()
        d = xc.shape[-1]
        n_tok = xc.numel() // d
        r = torch.empty(xc.shape[:-1] + (1,), device=xc.device, dtype=torch.float32)
        with torch.cuda.device(xc.device):
            check(_lib.lib().lb_rstd_fwd(ptr(xc), ptr(r), n_tok, d, float(eps), dtype_code(xc.dtype), stream_ptr()),
                  "rstd")
        ctx.save_for_backward(xc, r)
        return r

    @staticmethod
    def backward(ctx, gr: torch.Tensor):
        xc, r = ctx.saved_tensors
        d = xc.shape[-1]
        n_tok = xc.numel() // d
        gx = torch.empty_like(xc)
        grc = gr.contiguous().float()
        with torch.cuda.device(xc.device):
            check(_lib.lib().lb_rstd_bwd(ptr(xc), ptr(r), ptr(grc), ptr(gx), n_tok, d, dtype_code(xc.dtype),
                                         stream_ptr()), "rstd backward")
        return gx, None


def rstd(delta: torch.Tensor, eps: float) -> torch.Tensor:
    """The RMSNorm scale of a source, (b, t, 1) fp32, differentiable: the key of the read is delta * rstd."""
    _require_cuda(delta, "rstd")
    return _Rstd.apply(delta, float(eps))


def fused_read_supported(base, values, rstds, cbar) -> bool:
    """CUDA, contiguous, same-shape same-dtype bf16/fp32 sources and base; contiguous fp32 (b, t, 1) rstds and a
    contiguous fp32 (b, t, n) cbar.  Same predicate as the reference (fused_dattn.py:379-395), plus the kernels' own
    limits (row size a multiple of 16 bytes, at most 128 sources)."""
    v0 = values[0]
    if not v0.is_cuda or v0.dtype not in (torch.bfloat16, torch.float32):
        return False
    shape = v0.shape
    if base.dtype != v0.dtype or base.shape != shape:
        return False
    for v in values:
        if v.dtype != v0.dtype or v.shape != shape or not v.is_contiguous():
            return False
    rshape = shape[:-1] + (1,)
    for r in rstds:
        if r.dtype != torch.float32 or r.shape != rshape or not r.is_contiguous():
            return False
    if (shape[-1] * v0.element_size()) % 16 != 0 or shape[-1] * v0.element_size() > 16384:
        return False
    if len(values) > _lib.LB_MAX_SOURCES:
        return False
    return cbar.dtype == torch.float32 and cbar.shape == shape[:-1] + (len(values),) and cbar.is_contiguous()


# --------------------------------------------------------------------------------------------------------------
# shared launch helpers
# --------------------------------------------------------------------------------------------------------------
def _launch_read_fwd(V, R, dots, qi, base, cbar, c0, n_tok, d, N, n, save):
    dev = V.device
    out = torch.empty_like(base)
    tc = torch.empty((n_tok, n), device=dev, dtype=torch.float32)
    lg = lse = lse0 = None
    if save:
        lg = torch.empty((n_tok, n), device=dev, dtype=torch.float32)
        lse = torch.empty(n_tok, device=dev, dtype=torch.float32)
        lse0 = torch.empty(n_tok, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev), _timed("read_fwd", n, n + 2):
        check(_lib.lib().lb_read_fwd(ptr(V), ptr(R), ptr(dots), int(qi), ptr(base), ptr(cbar), ptr(c0), ptr(out),
                                     ptr(tc), ptr(lg), ptr(lse), ptr(lse0), n_tok, d, N, n, dtype_code(V.dtype),
                                     stream_ptr()), "read forward")
    return out, tc, lg, lse, lse0


def _scratch_for(d: int, device) -> torch.Tensor:
    nbytes = int(_lib.lib().lb_read_bwd_scratch_bytes(int(d)))
    return torch.empty(nbytes // 4, device=device, dtype=torch.float32)


# Optional timing hook: a callable(kind, n, units) -> context manager wrapped around the big launches; the benchmark
# installs one that brackets each launch with CUDA events on the launching stream. `units` is the number of
# [n_tok, d] row-vector transfers the launch makes by design (reads + writes). None = no overhead.
LAUNCH_TIMER = None


class _NoTimer:
    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


def _timed(kind, n, units):
    return _NoTimer() if LAUNCH_TIMER is None else LAUNCH_TIMER(kind, n, units)


def _bwd_units(n, accum, finalize, extra=0):
    """V once, the gradient stack read + written (written only on a first backward), g in, and with `finalize` the
    negated copy out."""
    return n + (2 * n if accum else n) + 1 + (1 if finalize else 0) + extra


def _launch_read_bwd(V, R, dV, dR, qc, g, gt, cbar, c0, lg, lse, lse0, scratch, n_tok, d, N, n, accum,
                     finalize=False, neg_out=None):
    """One backward read. With `finalize` the kernel also completes dV[n - 1] (adds the gradient that reaches the
    update through its key scale) and writes its negation to `neg_out`."""
    dev = V.device
    dcbar = torch.empty((n_tok, n), device=dev, dtype=torch.float32)
    dq = torch.empty(d, device=dev, dtype=torch.float32)
    with torch.cuda.device(dev), _timed("read_bwd", n, _bwd_units(n, accum, finalize)):
        if finalize:
            check(_lib.lib().lb_read_bwd_final(ptr(V), ptr(R), ptr(dV), ptr(dR), ptr(qc), ptr(g), ptr(gt), ptr(cbar),
                                               ptr(c0), ptr(lg), ptr(lse), ptr(lse0), ptr(dcbar), ptr(dq),
                                               ptr(scratch), ptr(neg_out), n_tok, d, N, n, int(bool(accum)),
                                               dtype_code(V.dtype), stream_ptr()), "read backward (final)")
        else:
            check(_lib.lib().lb_read_bwd(ptr(V), ptr(R), ptr(dV), ptr(dR), ptr(qc), ptr(g), ptr(gt), ptr(cbar),
                                         ptr(c0), ptr(lg), ptr(lse), ptr(lse0), ptr(dcbar), ptr(dq), ptr(scratch),
                                         n_tok, d, N, n, int(bool(accum)), dtype_code(V.dtype), stream_ptr()),
                  "read backward")
    return dq, dcbar


# --------------------------------------------------------------------------------------------------------------
# list layout: one tensor per source                                reference: fused_dattn.py:264-334
# --------------------------------------------------------------------------------------------------------------
class _ListStack:
    """The list layout's hidden stack. The kernels index ONE array of sources; a caller of the list layout holds one
    tensor per source and passes the same growing list read after read (the port model's loop). Instead of gathering
    all n sources again at every read, the sources seen so far are kept here: a read copies only the ones it has not
    seen (normally one, the newest), so a pass makes N row copies, not N^2 / 2. A slot is valid while the caller's
    tensor still has the address and the version it had when it was copied; anything else starts a new stack.
    Dropped when the first source is garbage-collected (the caller's pass is over) -- reads that still need it for
    their backward hold their own reference."""
    __slots__ = ("V", "R", "tags", "__weakref__")

    def __init__(self, cap, n_tok, d, dtype, device):
        self.V = torch.empty((cap, n_tok, d), dtype=dtype, device=device)
        self.R = torch.empty((cap, n_tok), dtype=torch.float32, device=device)
        self.tags = []                        # per filled slot: (value ptr, value version, scale ptr, scale version)

    @staticmethod
    def tag(v, r):
        return (v.data_ptr(), v._version, r.data_ptr(), r._version)


_LIST_STACKS = {}                             # (address of the first source, shape, dtype) -> _ListStack


def _list_stack(values, rstds):
    import weakref
    v0 = values[0]
    n, d = len(values), v0.shape[-1]
    n_tok = v0.numel() // d
    key = (v0.data_ptr(), tuple(v0.shape), v0.dtype, v0.device)
    ls = _LIST_STACKS.get(key)
    tags = [_ListStack.tag(v, r) for v, r in zip(values, rstds)]
    if ls is not None and (len(ls.tags) > n or ls.tags != tags[:len(ls.tags)]):
        ls = None                             # not the list this stack was built from
    if ls is None or ls.V.shape[0] < n:
        cap = max(8, 2 * n) if ls is not None else max(4, n)
        grown = _ListStack(min(cap, _lib.LB_MAX_SOURCES), n_tok, d, v0.dtype, v0.device)
        if ls is not None:
            k = len(ls.tags)
            grown.V[:k].copy_(ls.V[:k])
            grown.R[:k].copy_(ls.R[:k])
            grown.tags = list(ls.tags)
        ls = grown
        _LIST_STACKS[key] = ls
        weakref.finalize(v0, lambda k=key, ref=weakref.ref(ls): _LIST_STACKS.pop(k, None)
                         if _LIST_STACKS.get(k) is ref() else None)
    for i in range(len(ls.tags), n):
        ls.V[i].copy_(values[i].detach().reshape(n_tok, d))
        ls.R[i].copy_(rstds[i].detach().reshape(n_tok))
        ls.tags.append(tags[i])
    return ls


class FusedDattnRead(torch.autograd.Function):
    """(out, tc) = FusedDattnRead.apply(q, base, cbar, c0, *values, *rstds).

    The kernels index one stack; the list's sources are kept in a hidden one that persists from read to read, so each
    source is copied once per pass (see _ListStack). The stacked layout below needs no copy at all and accumulates
    the sources' gradients in the kernels; it is the path the trainer uses."""

    @staticmethod
    def forward(ctx, q, base, cbar, c0, *srcs):
        n = len(srcs) // 2
        values, rstds = srcs[:n], srcs[n:]
        cbar_c = cbar.detach().float().contiguous()
        if not fused_read_supported(base, values, rstds, cbar_c):
            raise RuntimeError("loopback_b200.FusedDattnRead: unsupported layout (see fused_read_supported)")
        v0 = values[0]
        d = v0.shape[-1]
        n_tok = v0.numel() // d
        dev = v0.device
        ls = _list_stack(values, rstds)
        N = ls.V.shape[0]
        qc = q.detach().float().contiguous()
        c0c = c0.detach().float().contiguous()
        base_c = base.detach().contiguous()
        dots = torch.empty((N, n_tok), device=dev, dtype=torch.float32)
        with torch.cuda.device(dev):
            check(_lib.lib().lb_scores(ptr(ls.V), ptr(qc), ptr(dots), n_tok, d, N, n, dtype_code(ls.V.dtype),
                                       stream_ptr()), "scores")
        save = any(ctx.needs_input_grad)         # no graph (inference): the backward's saves are not written
        out, tc, lg, lse, lse0 = _launch_read_fwd(ls.V, ls.R, dots, 0, base_c, cbar_c, c0c, n_tok, d, N, n, save=save)
        if save:
            ctx.save_for_backward(qc, cbar_c, c0c, lg, lse, lse0)
            ctx.ls = ls           # not a saved tensor: later reads append to the same stack (slots below n never change)
        ctx.n, ctx.q_dtype, ctx.base_shape = n, q.dtype, base.shape
        ctx.rshape = rstds[0].shape
        return out, tc.view(*base.shape[:-1], n)

    @staticmethod
    def backward(ctx, g, gt):
        qc, cbar_c, c0c, lg, lse, lse0 = ctx.saved_tensors
        ls, n = ctx.ls, ctx.n
        ctx.ls = None
        N, n_tok, d = ls.V.shape
        g = g.contiguous()
        gt_c = None if gt is None else gt.reshape(n_tok, n).float().contiguous()
        # the gradients of this read's sources: a private stack with the hidden stack's slice pitch
        dVt = torch.empty((n,) + tuple(ctx.base_shape), dtype=ls.V.dtype, device=ls.V.device)
        dRt = torch.empty((n, n_tok), dtype=torch.float32, device=ls.V.device)
        scratch = _scratch_for(d, ls.V.device)
        dq, dcbar = _launch_read_bwd(ls.V, ls.R, dVt, dRt, qc, g, gt_c, cbar_c, c0c, lg, lse, lse0, scratch, n_tok, d, N, n,
                                     accum=False)
        return (dq.to(ctx.q_dtype), g, dcbar.view(*ctx.base_shape[:-1], n), None,
                *dVt.unbind(0), *[dRt[i].view(ctx.rshape) for i in range(n)])


# --------------------------------------------------------------------------------------------------------------
# stacked layout                                                    reference: fused_dattn.py:398-409, :629-793
# --------------------------------------------------------------------------------------------------------------
def _alias(stack_tensor: torch.Tensor, s: int) -> torch.Tensor:
    """Slice s of a stack as a tensor that shares its storage but is not an autograd view of it: later slices are
    written in place, and autograd forbids a custom Function to return a view whose base is then modified."""
    sl = stack_tensor[s]
    out = torch.empty(0, dtype=stack_tensor.dtype, device=stack_tensor.device)
    out.set_(stack_tensor.untyped_storage(), sl.storage_offset(), sl.shape, sl.stride())
    return out


class DattnStack:
    """The stacked storage of one forward pass: V[n_steps, b, t, d] (the updates), R[n_steps, b, t, 1] (their key
    scales) and, from the first backward on, their gradient stacks dV / dR.  Given `query` (the read queries,
    (n_steps - 1, d); read s uses row s - 1) each write also stores the update's scores against the queries of the
    reads that will see it, DOTS[query, update, token] fp32, and the reads use those; the queries are taken as they
    are when the stack is built, i.e. for one forward pass."""
    __slots__ = ("V", "R", "dV", "dR", "n_steps", "n_tok", "d", "eps", "Q", "QT", "DOTS", "r_done", "_scratch",
                 "fuse_final", "_scale_done", "_neg", "_last_write", "_dq", "_dh0", "_first_step", "_first_blend",
                 "d_done", "defer_writes", "_pending", "_small", "deferred_grads", "_da", "_G", "_Wt", "_KQt", "_dv0", "_Qp",
                 "_n_step_nodes", "peer_reduce")

    def __init__(self, n_steps: int, shape, dtype, device, query=None, eps: float = 1e-6):
        b, t, d = shape
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("loopback_b200.DattnStack: device must be a CUDA device (there is no CPU path)")
        dtype_code(dtype)
        if (d * torch.empty(0, dtype=dtype).element_size()) % 16 != 0:
            raise RuntimeError(f"loopback_b200.DattnStack: row size of d={d} {dtype} is not a multiple of 16 bytes")
        if n_steps > _lib.LB_MAX_SOURCES:
            raise RuntimeError(f"loopback_b200.DattnStack: at most {_lib.LB_MAX_SOURCES} steps, got {n_steps}")
        self.n_steps, self.n_tok, self.d = int(n_steps), b * t, d
        self.V = torch.empty((n_steps, b, t, d), dtype=dtype, device=device)
        self.R = torch.empty((n_steps, b, t, 1), dtype=torch.float32, device=device)
        self.dV = self.dR = None
        self.eps = float(eps)
        self.r_done = [False] * self.n_steps      # R[s] written by the write of s
        self.d_done = [False] * self.n_steps      # ... and the scores of update s (DOTS[:, s, :])
        # Decode-sized batches without autograd: with defer_writes a write only records its tensors, and the read that
        # follows launches ONE kernel for both (lb_step_fwd). The tensor write() returned is filled by that launch,
        # not before; anything else that touches the stack first (another write, rstd, a read through another entry
        # point, flush()) performs the recorded write on its own.
        self.defer_writes = False
        self._pending = None
        self._small = b * t <= 4 * torch.cuda.get_device_properties(device).multi_processor_count
        self.Q = self.QT = self.DOTS = None
        self._scratch = None
        # The backward of read s is the last kernel to touch update s, so it also finishes that update's gradient
        # (the key-scale term, and the negated copy the write hands to the block input) instead of leaving them to
        # two more passes over it: _scale_done[s] / _neg[s] record what it did for the nodes that follow.
        self.fuse_final = True
        self._scale_done = [False] * self.n_steps
        self._neg = [None] * self.n_steps
        # Bookkeeping of the one-node-per-step path (FusedStepStk): the tensors of the newest write until the read
        # that follows it picks them up; the pass's query-gradient rows and loop-input gradient, which the steps'
        # backward kernels fill in place and the earliest step hands to autograd once.
        self._last_write = None
        self._dq = self._dh0 = None
        self._first_step = self._first_blend = None
        # Deferred gradient accumulation (lb_step_bwd_deferred): when every step of the pass is a FusedStepStk node and
        # the backward starts at the last step, no gradient stack dV is kept at all; each step's backward stores its
        # upstream gradient (_G, a stack like V) and two scalars per older source (_Wt, _KQt) and forms the finished
        # gradient of its own update from what the later steps left. Decided by the pass's first backward (_da).
        self.deferred_grads = True
        self._da = None
        self._G = self._Wt = self._KQt = self._dv0 = self._Qp = None
        self._n_step_nodes = 0
        # a dist.PeerQueryGrad: the step nodes then write their query-gradient rows into its peer-addressable buffer and
        # the pass's last backward returns the sum over the ranks (no collective is left to the caller)
        self.peer_reduce = None
        if query is not None:
            self.Q = query.detach().float().contiguous()
            self.DOTS = torch.empty((max(1, self.Q.shape[0]), self.n_steps, b * t), dtype=torch.float32, device=device)

    def write(self, s: int, h: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        """V[s] = h - x, returned as the update tensor (sharing the stack's storage, with the autograd edge to h
        and x)."""
        self.flush()
        if (self.defer_writes and self._small and 1 <= s < self.n_steps and not torch.is_grad_enabled()
                and h.dtype == self.V.dtype == x.dtype and h.shape == self.V.shape[1:] == x.shape
                and h.is_contiguous() and x.is_contiguous()):
            self._pending = (int(s), h, x)
            return self.V[s]                  # no autograd here: a plain view will do
        return _WriteDelta.apply(self, s, h, x)

    def flush(self) -> None:
        """Perform a write that was recorded for fusion with its read and has not been launched yet."""
        if self._pending is not None:
            s, h, x = self._pending
            self._pending = None
            with torch.no_grad():
                _WriteDelta.apply(self, s, h, x)

    def step_forward(self, step, h, x, h0, beta, tc_prev, lam, c0):
        """The recorded write of update `step` and the read that follows it as one launch (no autograd): returns
        (out, tc [n_tok, n])."""
        n, n_tok, d, dev = step + 1, self.n_tok, self.d, self.V.device
        self._pending = None
        out = torch.empty_like(h)
        tc = torch.empty((n_tok, n), device=dev, dtype=torch.float32)
        with _on(dev), _timed("step_fwd", n, n + 4 + (h0 is not None)):
            check(_lib.lib().lb_step_fwd(ptr(h), ptr(x), ptr(h0), float(beta), ptr(self.V), ptr(self.R), ptr(self.Q),
                                         ptr(tc_prev), float(lam), ptr(c0), ptr(out), ptr(tc), None, None, None, n_tok, d,
                                         self.n_steps, int(step), self.eps, dtype_code(self.V.dtype), stream_ptr()),
                  "step forward")
        self.r_done[step], self.d_done[step] = True, False
        return out, tc

    def rstd(self, s: int, delta: torch.Tensor, eps: float) -> torch.Tensor:
        """R[s] = the key scale of V[s], returned sharing the stack's storage (differentiable through `delta`)."""
        return _RstdStk.apply(self, s, delta, float(eps))

    def grads(self):
        if self.dV is None:
            self.dV = torch.empty_like(self.V)
            self.dR = torch.empty_like(self.R)
            return False
        return True

    def scratch(self) -> torch.Tensor:
        if self._scratch is None:
            self._scratch = _scratch_for(self.d, self.V.device)
        return self._scratch


class _WriteDelta(torch.autograd.Function):
    @staticmethod
    def forward(ctx, stack: DattnStack, s: int, h: torch.Tensor, x: torch.Tensor):
        if not 0 <= s < stack.n_steps:
            raise RuntimeError(f"delta_attnres stacked write: step {s} outside [0, {stack.n_steps})")
        if h.dtype != stack.V.dtype or x.dtype != stack.V.dtype:
            raise RuntimeError("delta_attnres stacked write: h and x must have the stack's dtype")
        if h.numel() != stack.n_tok * stack.d or x.numel() != stack.n_tok * stack.d:
            raise RuntimeError("delta_attnres stacked write: h and x must have the stack's shape")
        out = _alias(stack.V, s)
        hc, xc = h.detach().contiguous(), x.detach().contiguous()
        nq = 0 if stack.Q is None else stack.Q.shape[0]
        with torch.cuda.device(stack.V.device), _timed("write", s, 3):
            check(_lib.lib().lb_write(ptr(hc), ptr(xc), ptr(stack.V), ptr(stack.R), ptr(stack.Q), ptr(stack.DOTS),
                                      stack.n_tok, stack.d, stack.n_steps, nq, int(s), stack.eps,
                                      dtype_code(stack.V.dtype), stream_ptr()), "write")
        stack.r_done[s], stack.d_done[s] = True, nq > 0
        stack._last_write = (int(s), h, x)
        ctx.stack, ctx.s = stack, int(s)
        return out

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        stack, s = ctx.stack, ctx.s
        ctx.stack = None
        neg = stack._neg[s] if stack is not None else None
        if neg is not None:
            stack._neg[s] = None
            done = stack._dv0 if stack._da else (stack.dV[s] if stack.dV is not None else None)
            if stack._da:
                stack._dv0 = None
            if done is not None and g.data_ptr() == done.data_ptr() and g.shape == neg.shape:
                return None, None, g, neg            # the final read of update s already wrote -dV[s]
        gc = g.contiguous()
        dx = torch.empty_like(gc)
        with torch.cuda.device(gc.device):
            check(_lib.lib().lb_write_bwd_dx(ptr(gc), ptr(dx), gc.numel(), dtype_code(gc.dtype), stream_ptr()),
                  "write backward")
        return None, None, g, dx


class _RstdStk(torch.autograd.Function):
    @staticmethod
    def forward(ctx, stack: DattnStack, s: int, x: torch.Tensor, eps: float):
        stack.flush()
        r = _alias(stack.R, s)
        if not (stack.r_done[s] and eps == stack.eps):      # else the write already stored R[s]
            xc = x.detach().contiguous()
            with torch.cuda.device(xc.device):
                check(_lib.lib().lb_rstd_fwd(ptr(xc), ptr(r), stack.n_tok, stack.d, float(eps), dtype_code(xc.dtype),
                                             stream_ptr()), "stacked rstd")
        ctx.stack, ctx.s, ctx.x = stack, s, x
        return r

    @staticmethod
    def backward(ctx, gr: torch.Tensor):
        stack, s, x = ctx.stack, ctx.s, ctx.x
        if stack.dV is None and not stack._da:
            raise RuntimeError("delta_attnres stacked read: the scale's backward ran before any read's backward")
        grc = gr.contiguous().float()
        if stack._scale_done[s]:
            # the final read of update s already added the term for the gradient it produced itself (dR[s]); only a
            # gradient that reached the scale from elsewhere is still missing
            stack._scale_done[s] = False
            grc = None if grc.data_ptr() == stack.dR[s].data_ptr() else grc - stack.dR[s].reshape(grc.shape)
            if grc is not None:
                stack._neg[s] = None                 # the negated copy no longer matches
        if grc is not None:
            xc = x.detach().contiguous()
            dv_s = stack._dv0 if stack._da else stack.dV[s]
            with torch.cuda.device(xc.device):
                check(_lib.lib().lb_rstd_bwd_acc(ptr(xc), ptr(stack.R[s]), ptr(grc), ptr(dv_s), stack.n_tok, stack.d,
                                                 dtype_code(xc.dtype), stream_ptr()), "stacked rstd backward")
        if stack._da:                     # no gradient stack: update 0's gradient was handed over by the step-1 backward
            out = stack._dv0
        else:
            out = _alias(stack.dV, s)
        ctx.stack = ctx.x = None          # release the stack from this node
        return None, None, out, None


class FusedDattnReadStk(torch.autograd.Function):
    """(out, tc) = apply(stack, step, q, base, cbar, c0, *updates, *scales): the updates and scales are the stack's
    slices 0..step (inputs only for autograd's bookkeeping; the kernels read the stack)."""

    @staticmethod
    def forward(ctx, stack: DattnStack, step: int, q, base, cbar, c0, *srcs):
        n = len(srcs) // 2
        d, n_tok, dev = stack.d, stack.n_tok, stack.V.device
        if base.dtype != stack.V.dtype or not base.is_contiguous() or base.shape[:-1] != stack.V.shape[1:3]:
            raise RuntimeError("delta_attnres stacked read: base must be contiguous, the stack's dtype and shape")
        qc = q.detach().float().contiguous()
        c0c = c0.detach().float().contiguous()
        cbar_c = cbar.detach().float().contiguous()
        stack.flush()
        if stack.DOTS is not None and step >= 1 and all(stack.d_done[:n]):
            dots, qi = stack.DOTS, step - 1           # the stored scores of query step - 1 (q is that query)
        else:
            dots, qi = torch.empty((stack.n_steps, n_tok), device=dev, dtype=torch.float32), 0
            with torch.cuda.device(dev):
                check(_lib.lib().lb_scores(ptr(stack.V), ptr(qc), ptr(dots), n_tok, d, stack.n_steps, n,
                                           dtype_code(stack.V.dtype), stream_ptr()), "scores")
        save = any(ctx.needs_input_grad)         # no graph (inference): the backward's saves are not written
        out, tc, lg, lse, lse0 = _launch_read_fwd(stack.V, stack.R, dots, qi, base.detach(), cbar_c, c0c, n_tok, d,
                                                  stack.n_steps, n, save=save)
        if save:
            ctx.save_for_backward(qc, cbar_c, c0c, lg, lse, lse0)
        ctx.stack, ctx.step, ctx.n, ctx.q_dtype, ctx.base_shape = stack, int(step), n, q.dtype, base.shape
        # finish update `step` in this read's backward only if its key scale is part of the graph (it is when the
        # caller keeps the scales in `keys`, as both models do); otherwise nobody would consume the term
        ctx.finalize = bool(stack.fuse_final and save and ctx.needs_input_grad[6 + n + int(step)])
        return out, tc.view(*base.shape[:-1], n)

    @staticmethod
    def backward(ctx, g: torch.Tensor, gt):
        qc, cbar_c, c0c, lg, lse, lse0 = ctx.saved_tensors
        stack, step, n = ctx.stack, ctx.step, ctx.n
        d, n_tok = stack.d, stack.n_tok
        accum = stack.grads()
        g = g.contiguous()
        gt_c = None if gt is None else gt.reshape(n_tok, n).float().contiguous()
        neg = None
        if ctx.finalize:
            neg = torch.empty((n_tok, d), device=g.device, dtype=stack.V.dtype).view(stack.V.shape[1:])
            stack._scale_done[step], stack._neg[step] = True, neg
        dq, dcbar = _launch_read_bwd(stack.V, stack.R, stack.dV, stack.dR, qc, g, gt_c, cbar_c, c0c, lg, lse, lse0,
                                     stack.scratch(), n_tok, d, stack.n_steps, n, accum,
                                     finalize=ctx.finalize, neg_out=neg)
        final = [i == step or (step == 1 and i == 0) for i in range(n)]   # the last read of scale i, in backward order
        grads = (None, None, dq.to(ctx.q_dtype), g, dcbar.view(*ctx.base_shape[:-1], n), None,
                 *[None] * n, *[_alias(stack.dR, i) if final[i] else None for i in range(n)])
        # Release the stack from this node: ctx attributes live as long as the graph node, and a training loop that
        # keeps each micro-batch's loss until the optimizer step would otherwise keep every micro-batch's stack.
        ctx.stack = None
        return grads


class FusedCombineStk(torch.autograd.Function):
    """(out, tc) = apply(stack, step, q, proposal, h0, beta, tc_prev, lam, c0, *updates, *scales).

    FusedDattnReadStk with the cell's prologue folded into the kernels (LoopDeltaAttnRes.combine,
    looped_transformer.py:380-391): the installed coefficients are lam * (tc_prev, 1) and, when h0 is given (the
    read closes an iteration), base = proposal + beta (h0 - proposal). No base tensor, no coefficient tensor and
    none of the small torch kernels that built them exist any more; results are those of the unfused sequence."""

    @staticmethod
    def forward(ctx, stack, step, q, proposal, h0, beta, tc_prev, lam, c0, *srcs):
        n = len(srcs) // 2
        d, n_tok, dev = stack.d, stack.n_tok, stack.V.device
        for name, t in (("proposal", proposal), ("h0", h0)):
            if t is not None and (t.dtype != stack.V.dtype or not t.is_contiguous() or t.shape[:-1] != stack.V.shape[1:3]):
                raise RuntimeError(f"delta_attnres stacked read: {name} must be contiguous, the stack's dtype and shape")
        if n < 2 or tc_prev is None or tc_prev.shape[-1] != n - 1:
            raise RuntimeError("delta_attnres stacked read: the previous read's coefficients must have n - 1 entries")
        qc = q.detach().float().contiguous()
        c0c = c0.detach().float().contiguous()
        tcp = tc_prev.detach().float().contiguous()
        stack.flush()
        if stack.DOTS is not None and all(stack.d_done[:n]):
            dots, qi = stack.DOTS, step - 1
        else:
            dots, qi = torch.empty((stack.n_steps, n_tok), device=dev, dtype=torch.float32), 0
            with torch.cuda.device(dev):
                check(_lib.lib().lb_scores(ptr(stack.V), ptr(qc), ptr(dots), n_tok, d, stack.n_steps, n,
                                           dtype_code(stack.V.dtype), stream_ptr()), "scores")
        save = any(ctx.needs_input_grad)
        out = torch.empty_like(proposal)
        tc = torch.empty((n_tok, n), device=dev, dtype=torch.float32)
        lg = lse = lse0 = None
        if save:
            lg = torch.empty((n_tok, n), device=dev, dtype=torch.float32)
            lse = torch.empty(n_tok, device=dev, dtype=torch.float32)
            lse0 = torch.empty(n_tok, device=dev, dtype=torch.float32)
        with torch.cuda.device(dev), _timed("read_fwd", n, n + 2 + (h0 is not None)):
            check(_lib.lib().lb_combine_fwd(ptr(stack.V), ptr(stack.R), ptr(dots), int(qi), ptr(proposal.detach()),
                                            ptr(None if h0 is None else h0.detach()), float(beta), ptr(tcp), float(lam),
                                            ptr(c0c), ptr(out), ptr(tc), ptr(lg), ptr(lse), ptr(lse0), n_tok, d,
                                            stack.n_steps, n, dtype_code(stack.V.dtype), stream_ptr()), "combine forward")
        if save:
            ctx.save_for_backward(qc, tcp, c0c, lg, lse, lse0)
        ctx.stack, ctx.step, ctx.n, ctx.q_dtype, ctx.shape = stack, int(step), n, q.dtype, proposal.shape
        ctx.lam, ctx.beta, ctx.blend = float(lam), float(beta), h0 is not None
        ctx.finalize = bool(stack.fuse_final and save and ctx.needs_input_grad[9 + n + int(step)])
        return out, tc.view(*proposal.shape[:-1], n)

    @staticmethod
    def backward(ctx, g, gt):
        qc, tcp, c0c, lg, lse, lse0 = ctx.saved_tensors
        stack, step, n = ctx.stack, ctx.step, ctx.n
        d, n_tok, dev = stack.d, stack.n_tok, stack.V.device
        accum = stack.grads()
        g = g.contiguous()
        gt_c = None if gt is None else gt.reshape(n_tok, n).float().contiguous()
        neg = None
        if ctx.finalize:
            neg = torch.empty(stack.V.shape[1:], device=dev, dtype=stack.V.dtype)
            stack._scale_done[step], stack._neg[step] = True, neg
        dtc = torch.empty((n_tok, n - 1), device=dev, dtype=torch.float32)
        dq = torch.empty(d, device=dev, dtype=torch.float32)
        with torch.cuda.device(dev), _timed("read_bwd", n, _bwd_units(n, accum, ctx.finalize)):
            check(_lib.lib().lb_combine_bwd(ptr(stack.V), ptr(stack.R), ptr(stack.dV), ptr(stack.dR), ptr(qc), ptr(g),
                                            ptr(gt_c), ptr(tcp), ctx.lam, ptr(c0c), ptr(lg), ptr(lse), ptr(lse0),
                                            ptr(dtc), ptr(dq), ptr(stack.scratch()), ptr(neg), int(ctx.finalize), n_tok,
                                            d, stack.n_steps, n, int(bool(accum)), dtype_code(stack.V.dtype),
                                            stream_ptr()), "combine backward")
        dprop, dh0 = (g * (1.0 - ctx.beta), g * ctx.beta) if ctx.blend else (g, None)
        final = [i == step or (step == 1 and i == 0) for i in range(n)]
        grads = (None, None, dq.to(ctx.q_dtype), dprop, dh0, None, dtc.view(*ctx.shape[:-1], n - 1), None, None,
                 *[None] * n, *[_alias(stack.dR, i) if final[i] else None for i in range(n)])
        ctx.stack = None
        return grads


class FusedStepStk(torch.autograd.Function):
    """(out, tc) = apply(stack, step, query, h, x, h0, beta, tc_prev, lam, c0, *first): one autograd node for a whole
    step -- the write of update `step` (already done by stack.write(step, h, x), whose own node then never runs) and the
    read that follows it, with the cell's prologue inside the kernels as in FusedCombineStk.

    `query` is the whole (n_steps - 1, d) parameter, `h` / `x` the block's output / input, `h0` the loop input when the
    read closes an iteration (else None). `first` = (update 0, its key scale) for step 1, which also finishes update 0
    the way FusedDattnReadStk does; later steps take no update or scale as an input.

    The backward is one kernel plus the reduction of the query-gradient partials. It returns the step's own gradients:
    dL/dh = (the finished gradient of update `step`) + (the base's gradient), dL/dx = -(the update's gradient), so
    autograd has nothing to accumulate between the write and the read; the blend's factors are applied in the kernel
    (dL/dproposal = g - round(beta g), as autograd's own backward of h + beta (h0 - h) gives). Two gradients are built in
    place over the pass and handed to autograd once, by the earliest step (the last to run): the rows of the query
    gradient (each step's kernel writes row step - 1) and the loop input's gradient (accumulated in backward order
    with the storage dtype's rounding, like autograd's own accumulation)."""

    @staticmethod
    def forward(ctx, stack, step, query, h, x, h0, beta, tc_prev, lam, c0, *first):
        n = int(step) + 1
        d, n_tok, dev = stack.d, stack.n_tok, stack.V.device
        for name, t in (("h", h), ("h0", h0)):
            if t is not None and (t.dtype != stack.V.dtype or not t.is_contiguous() or t.shape[:-1] != stack.V.shape[1:3]):
                raise RuntimeError(f"delta_attnres stacked read: {name} must be contiguous, the stack's dtype and shape")
        if n < 2 or tc_prev is None or tc_prev.shape[-1] != n - 1:
            raise RuntimeError("delta_attnres stacked read: the previous read's coefficients must have n - 1 entries")
        c0c = c0.detach().float().contiguous()
        tcp = tc_prev.detach().float().contiguous()
        stack.flush()
        if stack.DOTS is not None and all(stack.d_done[:n]):
            dots, qi, qc = stack.DOTS, step - 1, stack.Q[step - 1]
        else:
            qc = query.detach()[step - 1].float().contiguous()
            dots, qi = torch.empty((stack.n_steps, n_tok), device=dev, dtype=torch.float32), 0
            with torch.cuda.device(dev):
                check(_lib.lib().lb_scores(ptr(stack.V), ptr(qc), ptr(dots), n_tok, d, stack.n_steps, n,
                                           dtype_code(stack.V.dtype), stream_ptr()), "scores")
        save = any(ctx.needs_input_grad)
        out = torch.empty_like(h)
        tc = torch.empty((n_tok, n), device=dev, dtype=torch.float32)
        lg = lse = lse0 = None
        if save:
            lg = torch.empty((n_tok, n), device=dev, dtype=torch.float32)
            lse = torch.empty(n_tok, device=dev, dtype=torch.float32)
            lse0 = torch.empty(n_tok, device=dev, dtype=torch.float32)
        with torch.cuda.device(dev), _timed("read_fwd", n, n + 2 + (h0 is not None)):
            check(_lib.lib().lb_combine_fwd(ptr(stack.V), ptr(stack.R), ptr(dots), int(qi), ptr(h.detach()),
                                            ptr(None if h0 is None else h0.detach()), float(beta), ptr(tcp), float(lam),
                                            ptr(c0c), ptr(out), ptr(tc), ptr(lg), ptr(lse), ptr(lse0), n_tok, d,
                                            stack.n_steps, n, dtype_code(stack.V.dtype), stream_ptr()), "combine forward")
        if save:
            ctx.save_for_backward(qc, tcp, c0c, lg, lse, lse0)
            stack._n_step_nodes += 1
            if stack._first_step is None:
                stack._first_step = int(step)
            if h0 is not None and ctx.needs_input_grad[5] and stack._first_blend is None:
                stack._first_blend = int(step)
        ctx.stack, ctx.step, ctx.n, ctx.shape = stack, int(step), n, h.shape
        ctx.q_dtype, ctx.q_rows = query.dtype, query.shape[0]
        ctx.lam, ctx.beta, ctx.blend = float(lam), float(beta), h0 is not None
        ctx.want_dh0 = bool(h0 is not None and ctx.needs_input_grad[5])
        ctx.n_first = len(first)
        return out, tc.view(*h.shape[:-1], n)

    @staticmethod
    def backward(ctx, g, gt):
        qc, tcp, c0c, lg, lse, lse0 = ctx.saved_tensors
        stack, step, n = ctx.stack, ctx.step, ctx.n
        d, n_tok, dev = stack.d, stack.n_tok, stack.V.device
        N = stack.n_steps
        if stack._da is None:                 # the pass's first backward decides how the updates' gradients are formed
            stack._da = bool(stack.deferred_grads and step == N - 1 and stack.dV is None and stack.dR is None
                             and stack._n_step_nodes == N - 1 and stack.Q is not None and stack.Q.shape[0] == N - 1)
        g = g.contiguous()
        gt_c = None if gt is None else gt.reshape(n_tok, n).float().contiguous()
        if stack._dq is None:
            if stack.peer_reduce is not None:
                if stack.peer_reduce.shape != (ctx.q_rows, d):
                    raise RuntimeError("delta_attnres stacked read: the peer reduction was built for another query shape")
                if stack._n_step_nodes != ctx.q_rows:
                    # a read that went another way hands its query-gradient row to autograd by itself, unsummed
                    raise RuntimeError("delta_attnres stacked read: the peer reduction of the query gradient needs every "
                                       f"read of the pass to be a fused step ({stack._n_step_nodes} of {ctx.q_rows} are)")
                stack._dq = stack.peer_reduce.rows.zero_()
            else:
                stack._dq = torch.zeros((ctx.q_rows, d), device=dev, dtype=torch.float32)
        dh0, dh0_accum = None, False
        if ctx.want_dh0:
            dh0_accum = stack._dh0 is not None
            if not dh0_accum:
                stack._dh0 = torch.empty(ctx.shape, device=dev, dtype=stack.V.dtype)
            dh0 = stack._dh0
        dh = torch.empty(ctx.shape, device=dev, dtype=stack.V.dtype)
        dx = torch.empty(ctx.shape, device=dev, dtype=stack.V.dtype)
        dtc = torch.empty((n_tok, n - 1), device=dev, dtype=torch.float32)
        dh0_units = (2 if dh0_accum else 1) if dh0 is not None else 0
        if stack._da:
            first = stack.dR is None
            if first:
                stack.dR = torch.empty_like(stack.R)
                stack._G = torch.empty_like(stack.V)
                stack._Wt = torch.empty((N, N, n_tok), device=dev, dtype=torch.float32)
                stack._KQt = torch.empty((N, N, n_tok), device=dev, dtype=torch.float32)
                code = dtype_code(stack.V.dtype)
                stack._Qp = torch.empty((N - 1, int(_lib.lib().lb_permuted_query_row_floats(d, code))), device=dev,
                                        dtype=torch.float32)
                with _on(dev):
                    check(_lib.lib().lb_permute_queries(ptr(stack.Q), ptr(stack._Qp), N - 1, d, code, stream_ptr()),
                          "permute queries")
            dv0 = dx0 = None
            if step == 1:                     # update 0 has no step of its own: this backward finishes it too
                dv0 = torch.empty(ctx.shape, device=dev, dtype=stack.V.dtype)
                dx0 = torch.empty(ctx.shape, device=dev, dtype=stack.V.dtype)
                stack._dv0, stack._neg[0], stack._scale_done[0] = dv0, dx0, True
            # g in and kept, V, the g rows of the later steps, dh and dx out (update 0: its row, those g rows again, 2 out)
            units = 1 + 1 + n + (N - n) + 2 + dh0_units + ((1 + (N - n) + 2) if step == 1 else 0)
            with _on(dev), _timed("read_bwd", n, units):
                check(_lib.lib().lb_step_bwd_deferred(
                    ptr(stack.V), ptr(stack.R), ptr(stack._G), ptr(stack.dR), ptr(stack._Wt), ptr(stack._KQt), ptr(stack.Q),
                    ptr(stack._Qp), ptr(g), ptr(gt_c), ptr(tcp), ctx.lam, ptr(c0c), ptr(lg), ptr(lse), ptr(lse0), ptr(dtc),
                    ptr(stack._dq[step - 1]), ptr(stack.scratch()), ptr(dh), ptr(dx), ptr(dh0), int(dh0_accum),
                    int(ctx.blend), ctx.beta, ptr(dv0), ptr(dx0), n_tok, d, N, n, int(first), dtype_code(stack.V.dtype),
                    stream_ptr()), "step backward (deferred)")
        else:
            accum = stack.grads()
            # V, the older updates' gradients (read + written), g and the newest update's gradient in, dh and dx out, the
            # loop input's gradient read + written at an iteration's end
            units = n + ((2 * (n - 1) + 1) if accum else (n - 1)) + 1 + 2 + dh0_units
            with _on(dev), _timed("read_bwd", n, units):
                check(_lib.lib().lb_step_bwd(ptr(stack.V), ptr(stack.R), ptr(stack.dV), ptr(stack.dR), ptr(qc), ptr(g),
                                             ptr(gt_c), ptr(tcp), ctx.lam, ptr(c0c), ptr(lg), ptr(lse), ptr(lse0), ptr(dtc),
                                             ptr(stack._dq[step - 1]), ptr(stack.scratch()), ptr(dh), ptr(dx), ptr(dh0),
                                             int(dh0_accum), int(ctx.blend), ctx.beta, n_tok, d, N, n,
                                             int(bool(accum)), dtype_code(stack.V.dtype), stream_ptr()), "step backward")
        dquery = dh0_out = None
        if step == stack._first_step:             # the earliest step runs last: the pass's query gradient is complete
            if stack.peer_reduce is not None:     # ... and is summed over the ranks here, through peer memory
                dquery, stack._dq = stack.peer_reduce.reduce().to(ctx.q_dtype), None
            else:
                dquery, stack._dq = stack._dq.to(ctx.q_dtype), None
        if ctx.want_dh0 and step == stack._first_blend:
            dh0_out, stack._dh0 = stack._dh0, None
        first = ()
        if ctx.n_first:                           # step 1 is also the last reader of update 0's key scale
            first = (None, _alias(stack.dR, 0))
        grads = (None, None, dquery, dh, dx, dh0_out, None, dtc.view(*ctx.shape[:-1], n - 1), None, None, *first)
        ctx.stack = None
        return grads


def device_error(clear: bool = True) -> int:
    """Synchronise and return the kernels' error word (0 = no bounded wait ran out); see lb_device_error."""
    return _lib.device_error(clear)

