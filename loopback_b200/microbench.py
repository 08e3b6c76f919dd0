"""Times ONE kernel of the library on synthetic data, through the C ABI, with CUDA events on the launching stream.

    python -m loopback_b200.microbench write    --tokens 32768 --d 1024 --N 24 --step 2      (22 queries scored)
    python -m loopback_b200.microbench read_fwd --tokens 32768 --d 1024 --N 24 --n 12 [--blend]
    python -m loopback_b200.microbench read_bwd --tokens 32768 --d 1024 --N 24 --n 12 [--first] [--blend]
    python -m loopback_b200.microbench step_bwd --tokens 32768 --d 1024 --N 24 --n 12 [--first] [--blend]
    python -m loopback_b200.microbench step_bwd_deferred --tokens 32768 --d 1024 --N 24 --n 12 [--blend]
    python -m loopback_b200.microbench step_fwd --tokens 64 --d 2048 --N 80 --n 40 --no-flush     (decode-sized)

Prints the average launch time, the row traffic the launch makes by design (GB) and the bandwidth that gives.
Between launches a buffer larger than L2 is rewritten (--no-flush turns that off), so every launch starts cold like
the launches of a real pass. The small cases this makes (one kernel, a handful of launches) are also what a profiler
capture of a single kernel should run.
"""
from __future__ import annotations

import argparse

import torch

from . import _lib as L


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["write", "read_fwd", "read_bwd", "step_bwd", "step_bwd_deferred", "step_fwd"])
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--d", type=int, default=1024)
    ap.add_argument("--N", type=int, default=24, help="updates of the pass (N - 1 queries)")
    ap.add_argument("--step", type=int, default=2, help="write: the update's index (queries max(step - 1, 0).. are scored)")
    ap.add_argument("--n", type=int, default=12, help="reads: the number of sources")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--first", action="store_true", help="backward: the pass's first backward (gradients written, not added)")
    ap.add_argument("--blend", action="store_true", help="the read closes an iteration (base blended with h0)")
    ap.add_argument("--bf16-queries", action="store_true", help="write: queries exactly representable in bf16")
    ap.add_argument("--no-scores", action="store_true", help="write: no queries (update and key scale only)")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--opt", action="append", default=[], help="library tuning knob name=value (lb_set_option)")
    a = ap.parse_args()

    lib = L.lib()
    for kv in a.opt:
        name, val = kv.split("=")
        L.set_option(name, int(val))
    dev = torch.device("cuda", torch.cuda.current_device())
    dt = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    code, elem = L.dtype_code(dt), (2 if a.dtype == "bf16" else 4)
    g = torch.Generator(device=dev).manual_seed(0)
    T, d, N, n = a.tokens, a.d, a.N, min(a.n, a.N)
    NQ = N - 1
    st = L.stream_ptr()

    def rnd(*shape, scale=1.0, dtype=dt):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(dtype)

    V = rnd(N, T, d, scale=0.3)
    R = torch.rsqrt(V[:, :, :64].float().pow(2).mean(-1) + 1e-6).contiguous()          # any positive scales do
    Q = rnd(NQ, d, scale=0.02, dtype=torch.float32)
    if a.bf16_queries:
        Q = Q.bfloat16().float()
    flush = None if a.no_flush else torch.empty(256 * 2**20, device=dev, dtype=torch.uint8)

    if a.kernel == "write":
        h, x = rnd(T, d), rnd(T, d)
        DOTS = torch.empty(NQ, N, T, device=dev)
        units, label = 3, f"write step {a.step}: {NQ - max(a.step - 1, 0)} queries scored"

        def launch():
            L.check(lib.lb_write(L.ptr(h), L.ptr(x), L.ptr(V), L.ptr(R), None if a.no_scores else L.ptr(Q), L.ptr(DOTS), T, d, N,
                                 NQ, a.step, 1e-6, code, st), "write")
    else:
        DOTS = rnd(N, T, scale=1.0, dtype=torch.float32)                                 # one query's block of scores
        c0 = (torch.rand(n, device=dev, generator=g) * 0.9 + 0.1).contiguous()
        tcp = (c0[:n - 1].view(1, -1) + 0.2 * torch.randn(T, n - 1, device=dev, generator=g)).contiguous()
        prop, h0 = rnd(T, d), rnd(T, d)
        out = torch.empty(T, d, device=dev, dtype=dt)
        tc, lg = torch.empty(T, n, device=dev), torch.empty(T, n, device=dev)
        lse, lse0 = torch.empty(T, device=dev), torch.empty(T, device=dev)
        lam = 0.25 if a.blend else 1.0

        def fwd():
            L.check(lib.lb_combine_fwd(L.ptr(V), L.ptr(R), L.ptr(DOTS), 0, L.ptr(prop), L.ptr(h0) if a.blend else None,
                                       0.75, L.ptr(tcp), lam, L.ptr(c0), L.ptr(out), L.ptr(tc), L.ptr(lg), L.ptr(lse),
                                       L.ptr(lse0), T, d, N, n, code, st), "combine forward")
        fwd()
        if a.kernel == "read_fwd":
            launch, units, label = fwd, n + 2 + int(a.blend), f"forward read, {n} sources"
        elif a.kernel == "step_fwd":
            hh, xx = rnd(T, d), rnd(T, d)
            units, label = n + 4 + int(a.blend), f"forward step (write + read, one launch), {n} sources"

            def launch():
                L.check(lib.lb_step_fwd(L.ptr(hh), L.ptr(xx), L.ptr(h0) if a.blend else None, 0.75, L.ptr(V), L.ptr(R),
                                        L.ptr(Q), L.ptr(tcp), lam, L.ptr(c0), L.ptr(out), L.ptr(tc), None, None, None, T, d,
                                        N, n - 1, 1e-6, code, st), "step forward")
        else:
            up, gt = rnd(T, d), torch.randn(T, n, device=dev, generator=g)
            dV, dR = rnd(N, T, d), torch.randn(N, T, device=dev, generator=g)
            dtc, dq = torch.empty(T, n - 1, device=dev), torch.empty(d, device=dev)
            scratch = torch.empty(lib.lb_read_bwd_scratch_bytes(d) // 4, device=dev)
            dh, dx = torch.empty(T, d, device=dev, dtype=dt), torch.empty(T, d, device=dev, dtype=dt)
            dh0 = rnd(T, d)
            accum = 0 if a.first else 1
            head = [L.ptr(V), L.ptr(R), L.ptr(dV), L.ptr(dR), L.ptr(Q[0]), L.ptr(up), L.ptr(gt), L.ptr(tcp), lam,
                    L.ptr(c0), L.ptr(lg), L.ptr(lse), L.ptr(lse0), L.ptr(dtc), L.ptr(dq), L.ptr(scratch)]
            if a.kernel == "step_bwd_deferred":
                G = dV                                   # the stack of upstream-gradient rows
                Wt = torch.randn(N, N, T, device=dev, generator=g) * 0.1
                KQt = torch.randn(N, N, T, device=dev, generator=g) * 0.01
                Qp = torch.empty(NQ, int(lib.lb_permuted_query_row_floats(d, code)), device=dev)
                L.check(lib.lb_permute_queries(L.ptr(Q), L.ptr(Qp), NQ, d, code, st), "permute queries")
                units = 2 + n + (N - n) + 2 + (2 if a.blend else 0)
                label = f"backward step (deferred), {n} sources of {N}{', blend' if a.blend else ''}"

                def launch():
                    L.check(lib.lb_step_bwd_deferred(L.ptr(V), L.ptr(R), L.ptr(G), L.ptr(dR), L.ptr(Wt), L.ptr(KQt), L.ptr(Q),
                                                     L.ptr(Qp), L.ptr(up), L.ptr(gt), L.ptr(tcp), lam, L.ptr(c0), L.ptr(lg), L.ptr(lse),
                                                     L.ptr(lse0), L.ptr(dtc), L.ptr(dq), L.ptr(scratch), L.ptr(dh), L.ptr(dx),
                                                     L.ptr(dh0) if a.blend else None, 1, int(a.blend), 0.75, None, None, T, d,
                                                     N, n, int(a.first), code, st), "step backward (deferred)")
            elif a.kernel == "read_bwd":
                units = n + (2 * n if accum else n) + 2
                label = f"backward read (finalising), {n} sources, {'accumulating' if accum else 'first'}"

                def launch():
                    L.check(lib.lb_combine_bwd(*head, L.ptr(dx), 1, T, d, N, n, accum, code, st), "combine backward")
            else:
                units = n + ((2 * (n - 1) + 1) if accum else (n - 1)) + 3 + (2 if a.blend else 0)
                label = f"backward step, {n} sources, {'accumulating' if accum else 'first'}{', blend' if a.blend else ''}"

                def launch():
                    L.check(lib.lb_step_bwd(*head, L.ptr(dh), L.ptr(dx), L.ptr(dh0) if a.blend else None, 1, int(a.blend),
                                            0.75, T, d, N, n, accum, code, st), "step backward")

    for _ in range(a.warmup):
        launch()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(a.iters):
        if flush is not None:
            flush.fill_(1)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    assert L.device_error() == 0, "a kernel gave up a bounded wait"
    ms = total / a.iters
    gb = units * T * d * elem / 1e9
    print(f"{label}: {T} tokens x d={d} {a.dtype}: {ms:.4f} ms per launch, {gb:.3f} GB by design ({units} rows per token), "
          f"{gb / (ms * 1e-3):.0f} GB/s")


if __name__ == "__main__":
    main()
