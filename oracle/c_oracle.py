"""ctypes binding of lb_oracle.c. TEST INFRASTRUCTURE, NOT PRODUCT (see the package docstring).

All arrays are C-contiguous numpy arrays of float32 or float64 (one flavour per call); bf16 storage is emulated by
values that are exactly representable in bf16, held in those arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liblb_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile lb_oracle.c with the Makefile beside it (gcc, OpenMP). Returns the library path."""
    src = os.path.join(_HERE, "lb_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liblb_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.lbo_round_bf16.restype = ctypes.c_float
        _lib.lbo_round_bf16.argtypes = [ctypes.c_float]
        _lib.lbo_num_threads.restype = ctypes.c_int
        for suf in ("f32", "f64"):
            getattr(_lib, f"lbo_chain_{suf}").restype = ctypes.c_int
    return _lib


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _suf(a: np.ndarray) -> str:
    if a.dtype == np.float32:
        return "f32"
    if a.dtype == np.float64:
        return "f64"
    raise TypeError(f"oracle arrays must be float32 or float64, got {a.dtype}")


def _chk(dt, *arrs):
    for a in arrs:
        if a is not None and (a.dtype != dt or not a.flags.c_contiguous):
            raise TypeError("oracle arrays must share one dtype and be C-contiguous")


def num_threads() -> int:
    return int(lib().lbo_num_threads())


def set_num_threads(n: int) -> None:
    lib().lbo_set_num_threads(ctypes.c_int(int(n)))


def round_bf16(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even to bf16, returned in the input's float type."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32).astype(a.dtype).reshape(a.shape)


def prior(step: int, num_blocks: int, beta: float):
    """(c0 [n], log-prior [n], mass) of read `step`, fp32, built by append-and-decay like the cell."""
    n = step + 1
    c0 = np.empty(n, np.float32)
    lc = np.empty(n, np.float32)
    mass = ctypes.c_float(0)
    lib().lbo_prior(ctypes.c_int(step), ctypes.c_int(num_blocks), ctypes.c_double(beta), _p(c0), _p(lc),
                    ctypes.byref(mass))
    return c0, lc, float(mass.value)


def write(h: np.ndarray, x: np.ndarray, eps: float, bf16_storage: bool):
    """(v [n_tok, d], r [n_tok]) of one update write."""
    suf = _suf(h)
    _chk(h.dtype, h, x)
    n_tok, d = h.shape
    v = np.empty_like(h)
    r = np.empty(n_tok, h.dtype)
    getattr(lib(), f"lbo_write_{suf}")(_p(h), _p(x), _p(v), _p(r), ctypes.c_int64(n_tok), ctypes.c_int(d),
                                       ctypes.c_double(eps), ctypes.c_int(int(bf16_storage)))
    return v, r


def base_blend(proposal: np.ndarray, h0: np.ndarray, beta: float, at_boundary: bool, bf16_storage: bool):
    suf = _suf(proposal)
    _chk(proposal.dtype, proposal, h0)
    out = np.empty_like(proposal)
    getattr(lib(), f"lbo_base_{suf}")(_p(proposal), _p(h0), _p(out), ctypes.c_int64(proposal.size),
                                      ctypes.c_double(beta), ctypes.c_int(int(at_boundary)),
                                      ctypes.c_int(int(bf16_storage)))
    return out


def read_fwd(V: np.ndarray, R: np.ndarray, q: np.ndarray, base: np.ndarray, cbar: np.ndarray, c0: np.ndarray,
             acc_bf16: bool = False, saves: bool = False):
    """One read. V [n, n_tok, d], R [n, n_tok], q [d], base [n_tok, d], cbar [n_tok, n], c0 [n] fp32.
    Returns (out, tc) or (out, tc, p, z) with saves=True."""
    suf = _suf(V)
    _chk(V.dtype, V, R, q, base, cbar)
    n, n_tok, d = V.shape
    c0 = np.ascontiguousarray(c0, np.float32)
    out = np.empty((n_tok, d), V.dtype)
    tc = np.empty((n_tok, n), V.dtype)
    p = np.empty((n_tok, n), V.dtype) if saves else None
    z = np.empty((n_tok, n), V.dtype) if saves else None
    getattr(lib(), f"lbo_read_fwd_{suf}")(_p(V), ctypes.c_int64(n_tok * d), _p(R), ctypes.c_int(n), _p(q), _p(base),
                                          _p(cbar), _p(c0), ctypes.c_int64(n_tok), ctypes.c_int(d),
                                          ctypes.c_int(int(acc_bf16)), _p(out), _p(tc), _p(p), _p(z))
    return (out, tc, p, z) if saves else (out, tc)


def read_bwd(V, R, q, cbar, c0, g, gt=None, want_dR: bool = False):
    """Gradients of one read: (dq [d], dV [n, n_tok, d] incl. the key-scale path, dcbar [n_tok, n][, dR [n, n_tok]])."""
    suf = _suf(V)
    _chk(V.dtype, V, R, q, cbar, g, gt)
    n, n_tok, d = V.shape
    c0 = np.ascontiguousarray(c0, np.float32)
    dq = np.zeros(d, V.dtype)
    dV = np.zeros_like(V)
    dcbar = np.empty((n_tok, n), V.dtype)
    dR = np.zeros((n, n_tok), V.dtype) if want_dR else None
    getattr(lib(), f"lbo_read_bwd_{suf}")(_p(V), ctypes.c_int64(n_tok * d), _p(R), ctypes.c_int(n), _p(q), _p(cbar),
                                          _p(c0), _p(g), _p(gt), ctypes.c_int64(n_tok), ctypes.c_int(d), _p(dq),
                                          _p(dV), _p(dcbar), _p(dR))
    return (dq, dV, dcbar, dR) if want_dR else (dq, dV, dcbar)


def chain(h0, D, Q, G, num_blocks: int, num_loops: int, beta: float, eps: float, bf16_storage: bool):
    """A whole K x R pass with blocks x -> x + D_s. h0 [n_tok, d], D [N, n_tok, d], Q [N-1, d], G [N, n_tok, d] or
    None. Returns dict(states [N, n_tok, d], tc_last [n_tok, N][, dq [N-1, d], dD [N, n_tok, d], dh0 [n_tok, d]])."""
    suf = _suf(h0)
    _chk(h0.dtype, h0, D, Q, G)
    n_tok, d = h0.shape
    N = num_blocks * num_loops
    states = np.empty((N, n_tok, d), h0.dtype)
    tc_last = np.empty((n_tok, N), h0.dtype)
    res = dict(states=states, tc_last=tc_last)
    dq = dD = dh0 = None
    if G is not None:
        dq = np.zeros((max(N - 1, 1), d), h0.dtype)
        dD = np.empty((N, n_tok, d), h0.dtype)
        dh0 = np.empty((n_tok, d), h0.dtype)
        res.update(dq=dq, dD=dD, dh0=dh0)
    rc = getattr(lib(), f"lbo_chain_{suf}")(_p(h0), _p(D), _p(Q), _p(G), ctypes.c_int64(n_tok), ctypes.c_int(d),
                                            ctypes.c_int(num_blocks), ctypes.c_int(num_loops), ctypes.c_double(beta),
                                            ctypes.c_double(eps), ctypes.c_int(int(bf16_storage)), _p(states),
                                            _p(tc_last), _p(dq), _p(dD), _p(dh0))
    if rc != 0:
        raise RuntimeError(f"lbo_chain failed with status {rc}")
    return res
