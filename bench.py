"""Benchmark of the Loopback read path: one step = one K x R pass (N writes, N-1 reads, the whole backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg2|cfg3|cfg4|cfg5] [--impl ours|reference]

Prints ONE JSON line. `value` is tokens/s of the headline workload (BASELINE configuration 2 unless --workload says
otherwise) with every input resident in HBM; `e2e` is the same pass with its inputs (h0, every block update, every
upstream gradient) copied from pinned host memory and its results (last state, query gradient) copied back inside the
timed region; `roofline` is the backward-read kernel's HBM bytes by design over its CUDA-event time against the
measured copy bandwidth; `cpu_baseline` is the CPU oracle (a C/OpenMP restatement of the reference read, not the
product) on a bounded token sample, timed on this host.

Beside the headline the line carries, under `config`:
  dropin_ms_per_step   the same pass through the reference-facing entry point (the cell's prologue in torch, then
                       FusedDattnReadStk.apply, as the reference trainer calls it);
  sharded              BASELINE configurations 3 and 4 with their FIXED token count split over the ranks of the run
                       (strong scaling; at --gpus 1 the whole configuration on one GPU), the query-gradient
                       all-reduce inside the timed region;
  depth_sweep          BASELINE configuration 5 (64 tokens, forward only) at R = 2, 4, 8, 16     (single-GPU runs);
  triton_reference     the reference's own Triton stack + cached-scores path on this GPU, same pass (single-GPU runs,
                       when a reference mirror is present under baseline/_ref/);
  torch_reference_gpu  the reference's PyTorch read on this GPU on a token sample.
Synthetic data only: h0 ~ N(0,1), updates ~ N(0,0.3^2), queries ~ N(0,0.02^2), upstream gradients ~ N(0,1).
With --gpus N > 1 (launched by torch.distributed.run) the headline is weak scaling (every rank runs one
configuration-2 shard); the only exchange is one all-reduce of the (N-1) x d query gradient per pass.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: d, K, R, batch, seq, storage dtype, backward?
    "cfg2": dict(d=1024, K=4, R=6, b=8, t=4096, dtype="bf16", backward=True),
    "cfg3": dict(d=1536, K=6, R=4, b=16, t=4096, dtype="bf16", backward=True),
    "cfg4": dict(d=3072, K=8, R=3, b=32, t=8192, dtype="bf16", backward=True),
    "cfg5": dict(d=2048, K=5, R=16, b=64, t=1, dtype="bf16", backward=False),
}
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 2**20


def algorithmic_units(N: int, backward: bool) -> int:
    """Row-vector transfers per token of one pass, in units of d * elem bytes: writes 3N; reads S + 2(N-1);
    backward S (V) + 2S - N (the gradient stack read + written, the first backward only writes) + (N-1) (g) + N
    (the block input's gradient, written by the read that finishes the update)."""
    S = N * (N + 1) // 2 - 1
    fwd = 3 * N + S + 2 * (N - 1)
    return fwd + (S + 2 * S - N + (N - 1) + N if backward else 0)


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:  # noqa: BLE001
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 50 ms from before the warm-up to the end of
    the run; `window()` brackets a timed region and `summary(window)` reports the samples that fell inside it."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index
        if index is None:
            return
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:  # noqa: BLE001
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append((time.monotonic(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            self.proc = None

    class _Window:
        def __enter__(self):
            self.t0 = time.monotonic()
            return self

        def __exit__(self, *a):
            self.t1 = time.monotonic()
            return False

    def window(self):
        return ClockSampler._Window()

    def summary(self, win):
        rows = [r for (ts, r) in self.rows if win.t0 <= ts <= win.t1 + 0.1 and len(r) >= 6]
        sm = [float(r[0]) for r in rows if r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if r[1].replace(".", "").isdigit()]
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [nm for k, nm in enumerate(names) if any(r[2 + k].lower() == "active" for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------------------------------------
# the reference arm / CPU baseline: the CPU oracle on a bounded token sample (never part of the measured product)
# ------------------------------------------------------------------------------------------------------------------
def cpu_pass_tokens_per_s(w, sample_tokens: int, repeats: int, warmup: int):
    import numpy as np

    from oracle import c_oracle as CO
    CO.build()
    CO.set_num_threads(os.cpu_count() or 1)      # all host cores, whatever OMP_NUM_THREADS the launcher exported
    N, d = w["K"] * w["R"], w["d"]
    rng = np.random.default_rng(0)
    h0 = rng.standard_normal((sample_tokens, d), dtype=np.float32)
    D = rng.standard_normal((N, sample_tokens, d), dtype=np.float32) * np.float32(0.3)
    Q = rng.standard_normal((N - 1, d), dtype=np.float32) * np.float32(0.02)
    G = rng.standard_normal((N, sample_tokens, d), dtype=np.float32) if w["backward"] else None
    bf16 = w["dtype"] == "bf16"
    if bf16:
        h0, D = CO.round_bf16(h0), CO.round_bf16(D)
    times = []
    for k in range(warmup + repeats):
        t0 = time.perf_counter()
        CO.chain(h0, D, Q, G, w["K"], w["R"], 0.75, 1e-6, bf16)
        if k >= warmup:
            times.append(time.perf_counter() - t0)
    return sample_tokens / statistics.median(times), statistics.median(times), CO.num_threads()


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = min(w["b"] * w["t"], 2048)
    tps, sec, cores = cpu_pass_tokens_per_s(w, sample, max(1, args.steps), max(1, args.warmup))
    line = {
        "impl": "reference", "metric": "loopback_read_fwd_bwd_tokens_per_s" if w["backward"] else "loopback_read_fwd_tokens_per_s",
        "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: d={w['d']} K={w['K']} R={w['R']} storage={w['dtype']}",
                   "sample": f"{sample} tokens of the {w['b'] * w['t']}-token workload (the read is token-parallel)"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} tokens, one K x R pass per step, C/OpenMP restatement of the reference read"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------------
# the measured arm
# ------------------------------------------------------------------------------------------------------------------
# dram__bytes_read.sum + dram__bytes_write.sum over the bytes by design of the captured launches (d=1024, bf16, 8192
# tokens; the summaries under profiles/ give the commands). Traffic grows in proportion to the tokens of a launch.
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = {"read_bwd": 0.99, "read_fwd": 1.004, "write": 0.845}


class Pass:
    """One K x R pass through the public entry points (DattnStack.write + LoopDeltaAttnRes.combine + autograd).
    `cell_factory(d, R, K)` / `stack_factory(cell, shape, dtype, dev)` let the same loop drive the reference's own
    modules (the Triton path, the PyTorch read) for the same-box comparison."""

    def __init__(self, w, device, seed, cell_factory=None, stack_factory=None, n_tok=None):
        import torch

        self.torch, self.w, self.dev = torch, w, device
        self.N, self.d = w["K"] * w["R"], w["d"]
        self.b, self.t = (w["b"], w["t"]) if n_tok is None else (1, n_tok)
        self.dtype = torch.bfloat16 if w["dtype"] == "bf16" else torch.float32
        g = torch.Generator(device=device).manual_seed(seed)
        shape = (self.b, self.t, self.d)
        if cell_factory is None:
            from loopback_b200.cell import LoopDeltaAttnRes
            self.cell = LoopDeltaAttnRes(self.d, w["R"], w["K"], beta=0.75, eps=1e-6).to(device)
            self.stack_factory = lambda cell, shp, dt, dev: cell.new_stack(shp, dt, dev, scores=True)
        else:
            self.cell = cell_factory(self.d, w["R"], w["K"]).to(device)
            self.stack_factory = stack_factory
        with torch.no_grad():
            self.cell.query.copy_(torch.randn(self.N - 1, self.d, device=device, generator=g) * 0.02)
        self.h0 = torch.randn(shape, device=device, generator=g).to(self.dtype).requires_grad_(w["backward"])
        # pools of 3 update / gradient tensors, cycled over the steps (kernel cost does not depend on the values)
        self.D = [(torch.randn(shape, device=device, generator=g) * 0.3).to(self.dtype) for _ in range(3)]
        self.G = [torch.randn(shape, device=device, generator=g).to(self.dtype) for _ in range(3)] if w["backward"] else None

    @property
    def n_tok(self):
        return self.b * self.t

    def run(self, h0=None, D=None, G=None):
        torch, cell, K = self.torch, self.cell, self.w["K"]
        h0 = self.h0 if h0 is None else h0
        D = self.D if D is None else D
        G = self.G if G is None else G
        backward = self.w["backward"]
        cell.query.grad = None
        h0.grad = None
        stack = None if self.stack_factory is None else self.stack_factory(cell, (self.b, self.t, self.d), self.dtype, self.dev)
        x, deltas, keys, coeffs, prior, outs = h0, [], [], None, None, []
        with torch.set_grad_enabled(backward):
            for s in range(self.N):
                l, blk = divmod(s, K)
                hs = x + D[s % len(D)]                       # the "block": harness cost, inside the timed region
                if stack is not None:
                    deltas.append(stack.write(s, hs, x))
                    x, coeffs, prior = cell.combine(hs, h0, deltas, coeffs, prior, l, blk, keys=keys, stack=stack)
                else:
                    deltas.append(hs - x)
                    x, coeffs, prior = cell.combine(hs, h0, deltas, coeffs, prior, l, blk, keys=keys)
                outs.append(x)
            if backward:
                torch.autograd.backward(outs, [G[s % len(G)] for s in range(self.N)])
        return x


class Runner:
    """Timing plumbing shared by every leg: barrier + synchronize on both sides, CUDA events on the launching stream,
    the maximum over ranks."""

    def __init__(self, torch, dist, dev, world):
        self.torch, self.dist, self.dev, self.world = torch, dist, dev, world

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def exchange(self, cell):
        """The pass's only exchange: the (N-1) x d query gradient summed over the ranks. With the peer reduction enabled
        on the cell, the pass's last backward has already done it (inside the captured graph too)."""
        if self.world > 1 and getattr(cell, "peer_reduce", None) is None:
            self.dist.all_reduce(cell.query.grad)

    def enable_peer(self, cell, mode):
        """Turn on the peer-memory reduction of the query gradient on every rank, or on none. Returns what is in use."""
        if self.world == 1 or mode != "peer":
            return "none" if self.world == 1 else "nccl all-reduce"
        try:
            cell.enable_peer_reduce(self.dev)
            ok, why = True, ""
        except Exception as e:  # noqa: BLE001 -- reported in the JSON line; the NCCL all-reduce takes over
            ok, why = False, f"{type(e).__name__}: {e}"[:160]
        if self.all_agree(ok):
            return "peer memory, one-shot (lb_peer_allreduce) as the last backward's epilogue"
        cell.__dict__["peer_reduce"] = None
        return "nccl all-reduce (peer memory unavailable" + (": " + why if why else " on another rank") + ")"

    def timed(self, fn, steps):
        torch = self.torch
        self.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        self.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(ms, op=self.dist.ReduceOp.MAX)
        return float(ms.item())

    def all_agree(self, ok: bool) -> bool:
        flag = self.torch.tensor([1 if ok else 0], device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(flag, op=self.dist.ReduceOp.MIN)
        return int(flag.item()) == 1

    def capture(self, P):
        """The pass as a CUDA graph (this rank's kernels only), or None when capture fails."""
        torch = self.torch
        try:
            side = torch.cuda.Stream(device=self.dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                P.run()                                      # allocator warm-up on the capture stream
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                P.run()
            return graph, None
        except Exception as e:  # noqa: BLE001 -- capture is an optimisation of the launch path only
            return None, type(e).__name__

    def measure(self, P, steps, warmup, graph=True, sampler=None):
        """Eager and (optionally) graph-replay time of a pass, the query-gradient all-reduce inside the timed region.
        Returns dict(ms, eager_ms, launch, clocks window)."""
        torch, dist, world = self.torch, self.dist, self.world
        backward = P.w["backward"]

        def eager_pass():
            P.run()
            if backward:
                self.exchange(P.cell)                        # the (N-1) x d query gradient: the only exchange
        for _ in range(warmup):
            eager_pass()
        win = sampler.window() if sampler is not None else ClockSampler._Window()
        with win:
            eager_ms = self.timed(eager_pass, steps) / steps
        res = dict(ms=eager_ms, eager_ms=eager_ms, launch="eager launches from Python", window=win)
        if graph:
            g, why = self.capture(P)
            if self.all_agree(g is not None):
                def graph_pass():
                    g.replay()
                    if backward:
                        self.exchange(P.cell)
                for _ in range(3):
                    graph_pass()
                win_g = sampler.window() if sampler is not None else ClockSampler._Window()
                with win_g:
                    graph_ms = self.timed(graph_pass, steps) / steps
                res["graph_ms"] = graph_ms
                if graph_ms < eager_ms:
                    res.update(ms=graph_ms, launch="CUDA graph replay of the whole pass", window=win_g)
            elif why:
                res["launch"] = f"eager launches from Python (graph capture failed: {why})"
            del g
        return res


def _release(torch):
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


def reference_legs(R, w, args, steps):
    """The reference's own code on this GPU, for the same-box comparison: its Triton stack + cached-scores path on the
    whole workload and its PyTorch read on a token sample. Needs the mirror under baseline/_ref/ (or $LOOPBACK_REF)."""
    torch = R.torch
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import stage_reference
        root = stage_reference.find()
    finally:
        sys.path.pop(0)
    if root is None:
        why = "no reference mirror (baseline/_ref/ or $LOOPBACK_REF) on this machine"
        return {"unavailable": why}, {"unavailable": why}
    from types import SimpleNamespace
    for p in (os.path.join(root, "trainer"), root):
        if p not in sys.path:
            sys.path.insert(0, p)
    triton_leg, torch_leg = None, None
    try:
        import flame.custom_models.looped_transformer.modeling_looped_transformer as MLT
        from flame.custom_models.looped_transformer import fused_dattn as TFD
        MLT._FUSED_DATTN = TFD
        P = Pass(w, R.dev, seed=0,
                 cell_factory=lambda d, Rr, K: MLT.LoopDeltaAttnRes(SimpleNamespace(hidden_size=d), Rr, K, beta=0.75, eps=1e-6),
                 stack_factory=lambda cell, shp, dt, dev: TFD.DattnStack(cell.num_steps, shp, dt, dev, query=cell.query, eps=cell.eps))
        m = R.measure(P, max(2, min(steps, 5)), 2, graph=False)
        triton_leg = {"ms_per_step": m["ms"], "tokens_per_s": P.n_tok / (m["ms"] * 1e-3), "launch": "eager launches (Triton JIT), "
                      "stack layout + cached scores (LOOP_DATTN_FUSED=1, LOOP_DATTN_STACK=1, LOOP_DATTN_DOTS=1)",
                      "what": "the reference's fused_dattn.py driven by the same pass on this GPU"}
        del P
        _release(torch)
    except Exception as e:  # noqa: BLE001 -- the comparison is optional; say why it is missing
        triton_leg = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    try:
        import looped_transformer as M
        M._FUSED_DATTN = False
        sample = min(w["b"] * w["t"], 4096)
        P = Pass(w, R.dev, seed=0, n_tok=sample,
                 cell_factory=lambda d, Rr, K: M.LoopDeltaAttnRes(d, Rr, K, beta=0.75, eps=1e-6), stack_factory=None)
        m = R.measure(P, max(2, min(steps, 5)), 2, graph=False)
        torch_leg = {"ms_per_step": m["ms"], "tokens_per_s": sample / (m["ms"] * 1e-3), "sample_tokens": sample,
                     "what": "the reference's PyTorch read (LoopDeltaAttnRes.combine, fused path off) on this GPU, "
                             "same pass on a token sample"}
        del P
        _release(torch)
    except Exception as e:  # noqa: BLE001
        torch_leg = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
    return triton_leg, torch_leg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only (no other configurations, no reference legs)")
    ap.add_argument("--tokens", type=int, default=0, help="override tokens per GPU (profiling on small cases)")
    ap.add_argument("--opt", action="append", default=[], help="library tuning knob name=value (lb_set_option)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="N > 1: how the query gradient is summed over the ranks (peer memory one-shot, or NCCL)")
    ap.add_argument("--no-graph", action="store_true", help="do not replay the pass as a CUDA graph for `value`")
    ap.add_argument("--path", default="fused", choices=["fused", "fused_combine", "dropin"],
                    help="how the headline pass calls the read (A/B): one node per step, prologue in the kernels, "
                         "or the reference-facing entry point")
    ap.add_argument("--detail", default="", help="write per-launch timings (kind, n, GB/s) to this file")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.tokens:
        w["b"], w["t"] = 1, args.tokens
    if args.impl == "reference":
        run_reference_arm(args, w)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist

    import loopback_b200._lib as L
    from loopback_b200 import fused_dattn as FD

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    L.lib()
    for kv in args.opt:
        name, val = kv.split("=")
        L.set_option(name, int(val))
    R = Runner(torch, dist, dev, world)

    N, d = w["K"] * w["R"], w["d"]
    n_tok = w["b"] * w["t"]
    elem = 2 if w["dtype"] == "bf16" else 4
    row = d * elem
    P = Pass(w, dev, seed=rank)

    peers = {}                                   # cell -> its PeerQueryGrad (only the one-node-per-step path uses it)

    def set_path(cell, path):
        cell.fuse_prologue = path in ("fused", "fused_combine")
        cell.fuse_step = path == "fused"
        if cell.peer_reduce is not None:
            peers[id(cell)] = cell.peer_reduce
        cell.__dict__["peer_reduce"] = peers.get(id(cell)) if path == "fused" else None
    exchange = R.enable_peer(P.cell, args.exchange) if w["backward"] else "none"
    set_path(P.cell, args.path)

    # ---- device-resident timing, with per-launch events on the dominant kernels -------------------------------
    sampler = ClockSampler(local if rank == 0 else None)       # rank 0 reports its own GPU's clocks
    launches = []

    class Timer:
        def __init__(self, kind, n, units):
            self.rec = (kind, n, units, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))

        def __enter__(self):
            self.rec[3].record()

        def __exit__(self, *a):
            self.rec[4].record()
            launches.append(self.rec)
            return False

    def one_pass():
        P.run()
        if w["backward"]:
            R.exchange(P.cell)
    for _ in range(args.warmup):
        one_pass()
    if world > 1 and P.cell.peer_reduce is not None and not R.all_agree(FD.device_error() == 0):
        # a rank's bounded wait for a peer ran out during warm-up (error 6): the NCCL all-reduce takes over on every rank
        P.cell.__dict__["peer_reduce"] = None
        peers.clear()
        args.exchange = "nccl"
        exchange = "nccl all-reduce (the peer-memory reduction gave up a wait during warm-up)"
        for _ in range(args.warmup):
            one_pass()
    FD.LAUNCH_TIMER = Timer
    count0 = L.LAUNCHES["count"]
    with sampler.window() as clocks:
        total_ms = R.timed(one_pass, args.steps)
    gpu_launches = (L.LAUNCHES["count"] - count0) // args.steps
    FD.LAUNCH_TIMER = None
    assert FD.device_error() == 0, "a kernel gave up a bounded wait"
    eager_ms_per_step = total_ms / args.steps
    ms_per_step, launch_mode = eager_ms_per_step, "eager launches from Python"

    # ---- the same pass captured once as a CUDA graph and replayed: removes the host's launch gaps. The capture holds
    # this rank's kernels only; the query-gradient all-reduce stays an ordinary call after each replay, and the
    # ranks agree (outside any capture) on whether every one of them captured successfully.
    graph = None
    if not args.no_graph:
        graph, why = R.capture(P)
        if why:
            launch_mode = f"eager launches from Python (graph capture failed: {why})"
        if R.all_agree(graph is not None):
            def graph_pass():
                graph.replay()
                if w["backward"]:
                    R.exchange(P.cell)
            for _ in range(3):
                graph_pass()
            assert FD.device_error() == 0
            with sampler.window() as clocks_g:
                graph_ms = R.timed(graph_pass, args.steps) / args.steps
            assert FD.device_error() == 0, "a kernel gave up a bounded wait"
            if graph_ms < ms_per_step:
                ms_per_step, launch_mode, clocks = graph_ms, "CUDA graph replay of the whole pass", clocks_g
    value = world * n_tok / (ms_per_step * 1e-3)

    # ---- the reference-facing entry point on the same pass: the prologue in torch, FusedDattnReadStk.apply -------
    dropin = None
    if not args.no_extras and args.path != "dropin":
        del graph
        graph = None
        set_path(P.cell, "dropin")
        m = R.measure(P, max(2, min(args.steps, 10)), 3, graph=not args.no_graph)
        dropin = {"ms_per_step": m["ms"], "eager_ms_per_step": m["eager_ms"], "launch": m["launch"]}
        set_path(P.cell, args.path)
        assert FD.device_error() == 0

    # ---- the harness's own share of a pass: the N block stand-ins h = x + D_s, timed alone (reported, not subtracted)
    hx, hd = P.h0.detach(), P.D[0].detach()
    hbuf = torch.empty_like(hx)                  # no allocation inside the timed loops

    def harness_adds():
        for _ in range(N):
            torch.add(hx, hd, out=hbuf)
    harness_adds()
    torch.cuda.synchronize()
    harness_ms = R.timed(harness_adds, 5) / 5
    # ... and autograd's own accumulations in the backward of that harness: every state feeds the next block, the next
    # write and the loss, so its gradient is the sum of three tensors (two adds per step)
    harness_bwd_ms = 0.0
    if w["backward"]:
        def harness_bwd_adds():
            for _ in range(2 * (N - 1)):
                torch.add(hx, hd, out=hbuf)
        harness_bwd_ms = R.timed(harness_bwd_adds, 5) / 5

    # ---- roofline of the dominant kernel: bytes by design of its launches over their event time -----------------
    peak, peak_kind = measured_peak()
    per_kind = {}
    for kind, n, units, a, b_ in launches:
        ms = a.elapsed_time(b_)
        acc = per_kind.setdefault(kind, [0.0, 0.0, 0])
        acc[0] += units * n_tok * row
        acc[1] += ms * 1e-3
        acc[2] += 1
    if args.detail and rank == 0:
        rows = {}
        for kind, n, units, a, b_ in launches:
            r = rows.setdefault((kind, n, units), [0.0, 0])
            r[0] += a.elapsed_time(b_)
            r[1] += 1
        with open(args.detail, "w") as f:
            f.write("kind n units launches ms_avg GBs frac_of_peak\n")
            for (kind, n, units), (ms, cnt) in sorted(rows.items()):
                gbs = units * n_tok * row / (ms / cnt * 1e-3) / 1e9
                f.write(f"{kind} {n} {units} {cnt} {ms / cnt:.4f} {gbs:.1f} {gbs / peak:.3f}\n")
    dominant = max(per_kind, key=lambda k: per_kind[k][1]) if per_kind else None
    roofline = None
    kernels = {}
    for kind, (by, sec, cnt) in per_kind.items():
        kernels[kind] = {"launches_per_step": cnt // args.steps, "ms_per_step": sec * 1e3 / args.steps,
                         "achieved_gbs": by / sec / 1e9, "frac": by / sec / 1e9 / peak}
    if dominant:
        by, sec, cnt = per_kind[dominant]
        roofline = {"bound": "hbm", "kernel": dominant, "achieved": by / sec / 1e9, "peak": peak, "unit": "GB/s",
                    "frac": by / sec / 1e9 / peak, "peak_source": peak_kind,
                    "traffic": (NCU_TRAFFIC_PER_ALGORITHMIC_BYTE[dominant] * by / cnt
                                if w["d"] == 1024 and w["dtype"] == "bf16" else None),
                    "traffic_source": "ncu dram bytes of an 8192-token capture of the same kernel and row size "
                                      "(profiles/step_bwd_deferred_cfg2_8192tok.md, read_fwd_cfg2_8192tok.md, "
                                      "write_mma_cfg2_32768tok.md), scaled by tokens",
                    "bytes_per_launch_avg": by / cnt, "ms_per_launch_avg": sec * 1e3 / cnt,
                    "note": "bytes by design of the launches that ran: the deferred step backward reads V (n rows), the "
                            "g rows of the later steps (N - n) and g, writes g, dh, dx -- N + 4 rows per token and step, "
                            "where the in-place form moves 3n + 2"}
    pass_units = algorithmic_units(N, w["backward"])
    pass_gbs = pass_units * n_tok * row / (ms_per_step * 1e-3) / 1e9
    # what this library's launches of one pass move by design (the sum of the launches' own row counts): less than the
    # formula above where the algorithm needs fewer transfers than the reference's (the deferred backward keeps no
    # gradient stack: N^2/2 row reads where the in-place accumulation makes N^2 transfers)
    design_units = sum(u for _, _, u, _, _ in launches) / max(1, args.steps)
    design_gbs = design_units * n_tok * row / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: host buffers in, results out, inside the timed region ------------------------------------
    e2e = None
    if not args.no_e2e and (N + 6) * n_tok * row > 32 * 2**30:
        print("bench: end-to-end leg skipped, its staging buffers would not fit beside the stacks", file=sys.stderr)
    elif not args.no_e2e:
        e2e = e2e_leg(R, P, w, args)

    # ---- the exchange alone, both ways (N > 1): the (N-1) x d query gradient summed over the ranks ----------------
    exchange_us = None
    if world > 1 and w["backward"]:
        qg = torch.randn(N - 1, d, device=dev)

        def per_call_us(fn, reps=20):
            """Device time of one call: `reps` calls captured as one CUDA graph (no host launch cost between them)."""
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            try:
                side = torch.cuda.Stream(device=dev)
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    fn()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for _ in range(reps):
                        fn()
                ok = True
            except Exception:  # noqa: BLE001 -- fall back to eager calls (host-bound: an upper bound)
                ok, g = False, None
            if R.all_agree(ok):
                g.replay()
                return R.timed(g.replay, 5) / 5 / reps * 1e3, "graph replay of 20 calls"
            return R.timed(fn, 50) / 50 * 1e3, "back-to-back eager calls (host-bound)"
        us, how = per_call_us(lambda: dist.all_reduce(qg))
        exchange_us = {"nccl_all_reduce": us, "nccl_how": how}
        pr = peers.get(id(P.cell)) or P.cell.peer_reduce
        if pr is not None:
            us, how = per_call_us(pr.reduce)
            exchange_us.update(peer_memory_one_shot=us, peer_how=how)
        exchange_us["what"] = "device time per call of the (N-1) x d fp32 sum alone, max over ranks"
        assert FD.device_error() == 0

    # ---- the other BASELINE configurations ------------------------------------------------------------------------
    sharded, depth_sweep, triton_leg, torch_leg = None, None, None, None
    if not args.no_extras:
        del P
        P = None
        _release(torch)
        sharded = {}
        for name in ("cfg3", "cfg4"):
            ws = dict(WORKLOADS[name])
            total = ws["b"] * ws["t"]
            per = total // world
            Ps = Pass(ws, dev, seed=rank, n_tok=per)
            R.enable_peer(Ps.cell, args.exchange)
            set_path(Ps.cell, args.path)
            # a graph keeps a second copy of the pass's memory alive: only where that fits comfortably
            use_graph = not args.no_graph and per * ws["d"] * 2 * 24 * 8 < 60 * 2**30
            m = R.measure(Ps, 3 if name == "cfg4" else 5, 2, graph=use_graph)
            u = algorithmic_units(ws["K"] * ws["R"], True)
            gbs = u * per * ws["d"] * 2 / (m["ms"] * 1e-3) / 1e9
            sharded[name] = {"tokens_total": total, "tokens_per_gpu": per, "ms_per_step": m["ms"],
                             "eager_ms_per_step": m["eager_ms"], "launch": m["launch"],
                             "tokens_per_s": per * world / (m["ms"] * 1e-3),
                             "pass_algorithmic_gbs_per_gpu": gbs, "pass_frac_of_peak": gbs / peak,
                             "device_error": int(FD.device_error())}
            del Ps
            _release(torch)
        if world == 1:
            depth_sweep = depth_sweep_leg(R, dev, rank, args, set_path)
            if rank == 0:
                triton_leg, torch_leg = reference_legs(R, dict(WORKLOADS[args.workload]) if not args.tokens else w, args, args.steps)

    # ---- CPU baseline (rank 0, single-GPU runs only) --------------------------------------------------------------
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample = min(n_tok, 2048)
        tps, sec, cores = cpu_pass_tokens_per_s(w, sample, repeats=3, warmup=1)
        cpu = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": f"{sample} tokens of the workload, one K x R pass, {sec:.2f} s per pass; "
                         "C/OpenMP restatement of the reference read"}

    if rank == 0:
        stack_bytes = N * n_tok * row
        l2_note = (f"inputs larger than L2 (the update stack alone is {stack_bytes / 2**20:.0f} MiB per GPU)"
                   if stack_bytes > L2_BYTES else
                   f"the pass's whole working set ({stack_bytes / 2**20:.0f} MiB of updates) is smaller than L2 and is "
                   "written by the pass before it is read: L2 residency is the workload's own, nothing is flushed")
        harness_total = harness_ms + harness_bwd_ms
        line = {
            "metric": "loopback_read_fwd_bwd_tokens_per_s" if w["backward"] else "loopback_read_fwd_tokens_per_s",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{args.workload}: d={d} K={w['K']} R={w['R']} B={w['b']} T={w['t']} per GPU, "
                                   f"storage={w['dtype']}, fp32 arithmetic, stack + cached scores, "
                                   f"{'forward+backward' if w['backward'] else 'forward only'}",
                       "storage_dtype": w["dtype"], "tokens_per_gpu": n_tok, "l2": l2_note,
                       "parallelism": f"tokens x{world}" if world > 1 else "single GPU",
                       "query_grad_exchange": exchange, "query_grad_exchange_us": exchange_us,
                       "path": args.path, "launch": launch_mode, "eager_ms_per_step": eager_ms_per_step,
                       "pass_algorithmic_units_per_token": pass_units,
                       "pass_algorithmic_gbs": pass_gbs, "pass_frac_of_peak": pass_gbs / peak,
                       "pass_frac_denominator": f"{peak:.1f} GB/s ({peak_kind} copy bandwidth)",
                       "pass_units_formula": "3N + S + 2(N-1) + S + (2S-N) + (N-1) + N, S = N(N+1)/2 - 1: the transfers of "
                                             "the reference's algorithm (in-place gradient accumulation)",
                       "pass_design_units_per_token": design_units, "pass_design_gbs": design_gbs,
                       "pass_design_frac_of_peak": design_gbs / peak,
                       "harness_adds_ms_per_step": harness_ms, "harness_backward_adds_ms_per_step": harness_bwd_ms,
                       "pass_frac_of_peak_without_harness_adds":
                           pass_units * n_tok * row / ((ms_per_step - harness_total) * 1e-3) / 1e9 / peak,
                       "dropin_ms_per_step": dropin["ms_per_step"] if dropin else None, "dropin": dropin,
                       "sharded": sharded, "depth_sweep": depth_sweep,
                       "triton_reference": triton_leg, "torch_reference_gpu": torch_leg,
                       "kernels": kernels},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": gpu_launches,
            "clocks": sampler.summary(clocks),
        }
        print(json.dumps(line), flush=True)
    sampler.stop()
    if world > 1:
        dist.destroy_process_group()


def depth_sweep_leg(R, dev, rank, args, set_path):
    """Decode-style depth sweep (BASELINE configuration 5: 64 tokens, forward only) at R = 2, 4, 8, 16 as graph replays
    and as eager launches."""
    import loopback_b200.fused_dattn as FD
    torch = R.torch
    w5 = dict(WORKLOADS["cfg5"])
    out = []
    for r_iter in (2, 4, 8, 16):
        wr = dict(w5, R=r_iter)
        Pr = Pass(wr, dev, seed=rank)
        set_path(Pr.cell, args.path)
        m = R.measure(Pr, 20, 3, graph=not args.no_graph)
        n_r = wr["K"] * r_iter
        units = algorithmic_units(n_r, False)
        ms_r = m["ms"]
        out.append({"R": r_iter, "updates": n_r, "ms_per_pass": ms_r, "eager_ms_per_pass": m["eager_ms"],
                    "us_per_step": ms_r * 1e3 / n_r, "eager_us_per_step": m["eager_ms"] * 1e3 / n_r,
                    "algorithmic_gbs": units * Pr.n_tok * wr["d"] * 2 / (ms_r * 1e-3) / 1e9})
        assert FD.device_error() == 0
        del Pr
    _release(torch)
    return out


def e2e_leg(R, P, w, args):
    """The pass with host-fed inputs: h0, every update and every upstream gradient staged from pinned host memory on a
    copy stream, the last state and the query gradient copied back, all inside the timed region."""
    torch, dist, dev, world = R.torch, R.dist, R.dev, R.world
    N, d = P.N, P.d
    n_tok = P.n_tok
    elem = 2 if w["dtype"] == "bf16" else 4
    shape = (w["b"], w["t"], d)
    host_h0 = torch.randn(shape).to(P.dtype).pin_memory()
    host_D = [(torch.randn(shape) * 0.3).to(P.dtype).pin_memory() for _ in range(2)]
    host_G = [torch.randn(shape).to(P.dtype).pin_memory() for _ in range(2)] if w["backward"] else None
    out_host = torch.empty(shape, dtype=P.dtype).pin_memory()
    dq_host = torch.empty((N - 1, d), dtype=torch.float32).pin_memory()
    copy_stream = torch.cuda.Stream(device=dev)
    h2d = (1 + N + (N if w["backward"] else 0)) * n_tok * d * elem
    d2h = n_tok * d * elem + ((N - 1) * d * 4 if w["backward"] else 0)

    # Fixed device staging: a ring of 4 buffers for the updates (each is consumed by the step's first kernel), one
    # buffer per read for the upstream gradients (autograd reads them at times of its own choosing), two for h0.
    # All copies run on the copy stream in the order they are needed; a buffer is overwritten only after the
    # compute stream has passed the event that marks its last use, so neither the allocator nor stream-recording
    # is involved, and the next pass's copies overlap this pass's backward.
    ring = [torch.empty(shape, dtype=P.dtype, device=dev) for _ in range(4)]
    ring_free = [None] * len(ring)            # compute-stream events: the slot may be overwritten after them
    gbufs = [torch.empty(shape, dtype=P.dtype, device=dev) for _ in range(N)] if w["backward"] else None
    h0bufs = [torch.empty(shape, dtype=P.dtype, device=dev) for _ in range(2)]
    pass_done = [None, None]                  # end of the last pass that used h0bufs[k]
    last_done = {"ev": None, "count": 0}

    def stage_update(s):
        slot = s % len(ring)
        with torch.cuda.stream(copy_stream):
            if ring_free[slot] is not None:
                copy_stream.wait_event(ring_free[slot])
            ring[slot].copy_(host_D[s % len(host_D)], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        torch.cuda.current_stream().wait_event(ev)
        return ring[slot]

    def stage_grads():
        """All upstream gradients of the pass, last read first (the order the backward consumes them)."""
        with torch.cuda.stream(copy_stream):
            if last_done["ev"] is not None:
                copy_stream.wait_event(last_done["ev"])          # the previous pass no longer reads the buffers
            for s in range(N - 1, -1, -1):
                gbufs[s].copy_(host_G[s % len(host_G)], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(copy_stream)
        torch.cuda.current_stream().wait_event(ev)

    def e2e_pass():
        """Pass.run with host-fed inputs: the same calls, plus the staging copies and their events."""
        cur = torch.cuda.current_stream()
        k = last_done["count"] & 1
        with torch.cuda.stream(copy_stream):
            if pass_done[k] is not None:
                copy_stream.wait_event(pass_done[k])
            h0bufs[k].copy_(host_h0, non_blocking=True)
            ev0 = torch.cuda.Event()
            ev0.record(copy_stream)
        cur.wait_event(ev0)
        h0d = h0bufs[k].detach().requires_grad_(w["backward"])
        cell, K = P.cell, w["K"]
        cell.query.grad = None
        stack = cell.new_stack((w["b"], w["t"], d), P.dtype, dev, scores=True)
        x, deltas, keys, coeffs, prior, outs = h0d, [], [], None, None, []
        with torch.set_grad_enabled(w["backward"]):
            for s in range(N):
                l, blk = divmod(s, K)
                hs = x + stage_update(s)
                rel = torch.cuda.Event()
                rel.record(cur)
                ring_free[s % len(ring)] = rel
                deltas.append(stack.write(s, hs, x))
                x, coeffs, prior = cell.combine(hs, h0d, deltas, coeffs, prior, l, blk, keys=keys, stack=stack)
                outs.append(x)
            if w["backward"]:
                stage_grads()
                torch.autograd.backward(outs, [gbufs[s] for s in range(N)])
        if w["backward"]:
            R.exchange(cell)
        out_host.copy_(x.detach(), non_blocking=True)
        if w["backward"]:
            dq_host.copy_(cell.query.grad, non_blocking=True)
        done = torch.cuda.Event()
        done.record(cur)
        pass_done[k] = done
        last_done["ev"] = done
        last_done["count"] += 1

    for _ in range(2):
        e2e_pass()
    e2e_steps = max(2, min(args.steps, 5))
    e2e_ms = R.timed(e2e_pass, e2e_steps) / e2e_steps
    # for context: what this box's host link gives a plain pinned-memory copy of one such tensor, back to back
    torch.cuda.synchronize()

    def raw_copies():
        for k in range(8):
            ring[k % len(ring)].copy_(host_D[k % 2], non_blocking=True)
    raw_copies()
    h2d_gbs = 8 * n_tok * d * elem / (R.timed(raw_copies, 1) * 1e-3) / 1e9
    return {"value": world * n_tok / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "h2d_gbs_in_pass": h2d / (e2e_ms * 1e-3) / 1e9, "h2d_gbs_plain_copies": h2d_gbs,
            "note": "bound by the host link: compare the rate at which the pass moves its inputs (h2d_gbs_in_pass, with the "
                    "results going back at the same time) with what plain pinned-memory copies reach on this box"}


if __name__ == "__main__":
    main()
