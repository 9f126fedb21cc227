#!/usr/bin/env python
"""Benchmark of the circulant-attention hot path.

A step = one fused forward + backward of multi-head circulant attention over one
batch of synthetic input at the README quickstart shape (H, W, C, B = 128, 96,
64, 2; ws = 15; 4 heads; DotSimilarity + softmax; Float32), flash mode (A is not
written).  Metric: query pixels per second (one query pixel = one spatial
location of one batch element with all channels and heads).

    python bench.py [--gpus N --steps K --warmup W] [--impl reference]

`--impl reference` times the CPU restatement (C + OpenMP; the reference package
has no CPU path and cannot run without Julia) on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(H=128, W=96, C=64, B=2, ws=15, nheads=4)
METRIC = "fwd+bwd query-pixels/sec (ws=15, C=64, 4 heads)"
UNIT = "px/s"
NOMINAL_FFMA_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12


def algorithmic(workload, what):
    """Algorithmic flops and bytes per query pixel: Dot fwd 4*K*C, bwd 10*K*C flop;
    bytes fwd 4*C*4, bwd 7*C*4 (A not materialised)."""
    K, C = workload["ws"] ** 2, workload["C"]
    flops = {"fwd": 4 * K * C, "bwd": 10 * K * C, "bwd_dq": 6 * K * C, "bwd_dkdv": 4 * K * C}
    flops["fwd+bwd"] = flops["fwd"] + flops["bwd"]
    bytes_ = {"fwd": 16 * C, "bwd": 28 * C, "fwd+bwd": 44 * C, "bwd_dq": 20 * C, "bwd_dkdv": 28 * C}
    return flops[what], bytes_[what]


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.path = index, None, f"/tmp/circatt_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def wait_first_sample(self, limit_s=5.0):
        t0 = time.perf_counter()
        while self.proc is not None and time.perf_counter() - t0 < limit_s:
            try:
                if os.path.getsize(self.path) > 0:
                    return
            except OSError:
                pass
            time.sleep(0.01)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); smax.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None, "reasons": sorted(reasons), "samples": len(sm)}


# --------------------------------------------------------------------------- reference arm (CPU)
def make_inputs(workload, seed):
    rng = np.random.default_rng(seed)
    shape = (workload["H"], workload["W"], workload["C"], workload["B"])
    return [np.asfortranarray(rng.standard_normal(shape).astype(np.float32)) for _ in range(4)]


def cpu_step(cpu, orc, arrs, workload):
    q, k, v, r = (orc.splitheads(t, workload["nheads"]) for t in arrs)
    y, lse = cpu.attention_fwd(q, k, v, workload["ws"])
    return cpu.attention_bwd(q, k, v, y, r, lse, workload["ws"])


def run_cpu(workload, steps, warmup):
    from oracle import circatt_oracle as orc
    from oracle import cpu_baseline as cpu
    cpu.use_all_cores()              # launchers such as torchrun export OMP_NUM_THREADS=1
    arrs = make_inputs(workload, 0)
    for _ in range(warmup):
        cpu_step(cpu, orc, arrs, workload)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(cpu, orc, arrs, workload)
    dt = (time.perf_counter() - t0) / steps
    px = workload["H"] * workload["W"] * workload["B"]
    return px / dt, dt, cpu.threads()


def reference_main(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = max(1, min(args.steps, 20)), max(1, min(args.warmup, 3))
    value, dt, threads = run_cpu(WORKLOAD, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic (numpy default_rng(0) standard normal)",
        "config": {"workload": "circulant_mh_attention fwd+bwd, H,W,C,B=128,96,64,2, ws=15, 4 heads, Dot, softmax",
                   **WORKLOAD},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "the full step (24576 query pixels), C + OpenMP float32 restatement; "
                                   "the reference is Julia + CUDA.jl only and has no CPU path"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))



# --------------------------------------------------------------------------- other configurations
OTHER_CONFIGS = {
    # name: (Julia shape, ws, heads, similarity, normaliser, complex, A materialised, storage dtype)
    "c1": ((32, 32, 16, 1), 7, 1, 0, 0, False, True, "f32"),
    "c3": ((16384, 64, 16), 127, 8, 1, 1, False, False, "f32"),        # 1-D, Distance, entmax-1.5
    "c4": ((320, 320, 32, 8), 7, 1, 0, 0, True, True, "c64"),          # ComplexF32, A materialised
    "c5_one_batch_f32": ((1024, 1024, 128, 1), 21, 8, 0, 0, False, False, "f32"),
    "c5_one_batch_bf16": ((1024, 1024, 128, 1), 21, 8, 0, 0, False, False, "bf16"),
}


def config_flops(shape, ws, kind, cplx):
    """Algorithmic flops per query pixel (forward, backward): Dot 4*K*C / 10*K*C, Distance 5*K*C / 11*K*C,
    complex channels counted twice."""
    K = ws ** (len(shape) - 2)
    C = shape[-2] * (2 if cplx else 1)
    return (5 if kind else 4) * K * C, (11 if kind else 10) * K * C


def make_timer(torch, flush):
    def timed(fn, n=5, warm=2):
        for _ in range(warm):
            fn()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in evs:
            flush.fill_(1)
            a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(b) * 1e-3 for a, b in evs)
        return ts[len(ts) // 2]
    return timed


def time_config(ca, torch, timed, gen, cfg, ffma_tflops):
    """Forward and forward+backward of one BASELINE configuration through the ops layer (C ABI), device
    resident, L2 flushed before every timed call."""
    shape, ws, nh, kind, norm, cplx, want_nz, store = cfg
    ops, jl = ca.ops, ca.jl
    dt = torch.complex64 if cplx else torch.float32
    q, k, v, dy = (ca.splitheads(jl.randn(*shape, generator=gen, dtype=dt), nh) for _ in range(4))
    if store == "bf16":
        q, k, v, dy = (t.to(torch.bfloat16) for t in (q, k, v, dy))
    px = int(np.prod(shape[:-2])) * shape[-1]
    res = {}

    def fwd():
        res["r"] = ops.attention_fwd(kind, norm, q, k, v, ws, want_nz, keep_workspace=True)
    tf = timed(fwd)
    y, nz, stats, fws = res["r"]
    tb = timed(lambda: ops.attention_bwd(kind, norm, q, k, v, y, dy, stats, ws, nz=nz,
                                         fwd_workspace=fws if norm == 0 else None))
    fl_f, fl_b = config_flops(shape, ws, kind, cplx)
    out = {"fwd_us": tf * 1e6, "bwd_us": tb * 1e6, "fwd_px_per_s": px / tf, "fwd_bwd_px_per_s": px / (tf + tb),
           "fwd_tflops": px * fl_f / tf / 1e12, "bwd_tflops": px * fl_b / tb / 1e12,
           "roofline_frac_ffma": px * (fl_f + fl_b) / (tf + tb) / 1e12 / ffma_tflops}
    del q, k, v, dy, y, nz, stats, fws, res
    ops.release_scratch()
    torch.cuda.empty_cache()
    return out


# --------------------------------------------------------------------------- independent float64 check (torch)
def sampled_reference(torch, q, k, v, dy, ws, pixels, unit):
    """Float64 torch restatement of softmax circulant attention and its gradients at a few pixels of one
    unit: y[j] and dq[j] need the window of j; dk[i] and dv[i] need every query whose window holds i,
    each with its own window.  q, k, v, dy: (H, W, c, units) tensors of the FULL image.  Returns four
    (len(pixels), c) float64 tensors."""
    H, W, c = q.shape[0], q.shape[1], q.shape[2]
    p = (ws - 1) // 2
    scale = 1.0 / float(c) ** 0.5
    Q, Kk, V, DY = (t[..., unit].double() for t in (q, k, v, dy))
    d = torch.arange(-p, p + 1, device=q.device)

    def windows(hs, ws_):
        """key pixels of the queries (hs[n], ws_[n]): index tensors (n, K), w-major like the CSR order"""
        hh = (hs[:, None] + d[None, :]) % H                      # (n, ws)
        ww = (ws_[:, None] + d[None, :]) % W
        return hh[:, None, :].expand(-1, ws, -1).reshape(len(hs), -1), ww[:, :, None].expand(-1, -1, ws).reshape(len(hs), -1)

    def rows(hs, ws_):
        hh, ww = windows(hs, ws_)
        kw, vw = Kk[hh, ww], V[hh, ww]                           # (n, K, c)
        qs, dys = Q[hs, ws_], DY[hs, ws_]                        # (n, c)
        P = torch.softmax(scale * torch.einsum("nc,nkc->nk", qs, kw), dim=1)
        dP = torch.einsum("nc,nkc->nk", dys, vw)
        dS = P * (dP - (P * dP).sum(1, keepdim=True))
        return P, dS, kw, vw, hh, ww

    hs = torch.tensor([j % H for j in pixels], device=q.device)
    wcol = torch.tensor([j // H for j in pixels], device=q.device)
    P, dS, kw, vw, hh, ww = rows(hs, wcol)
    y = torch.einsum("nk,nkc->nc", P, vw)
    dq = scale * torch.einsum("nk,nkc->nc", dS, kw)
    dk, dv = torch.zeros_like(y), torch.zeros_like(y)
    for n in range(len(pixels)):
        # the queries that see pixel n are the pixels of its own window (window symmetry)
        hq, wq = hh[n], ww[n]
        Pq, dSq, _, _, hhq, wwq = rows(hq, wq)
        hit = (hhq == hs[n]) & (wwq == wcol[n])                  # position of pixel n inside each of those windows
        dk[n] = scale * ((dSq * hit).sum(1)[:, None] * Q[hq, wq]).sum(0)
        dv[n] = ((Pq * hit).sum(1)[:, None] * DY[hq, wq]).sum(0)
    return y, dq, dk, dv


def band_c5(ca, torch, dist, dev, world, rank, steps):
    """One 1024 x 1024 x 128 image of BASELINE config 5 (ws 21, 8 heads, flash mode) cut into bands of columns
    over the ranks: forward + backward with the halo exchanges (the circular wrap between the last and the
    first rank included) inside the timed region, and a float64 check of rank 0's band at border pixels."""
    jl, par = ca.jl, ca.parallel
    H, W, C, ws, nh = 1024, 1024, 128, 21, 8
    plan = par.BandPlan(W, world, ws)
    start, width = plan.band(rank)
    gen = torch.Generator(device=dev).manual_seed(1234)          # every rank draws the same full image
    full = [ca.splitheads(jl.randn(H, W, C, 1, generator=gen, device=dev), nh) for _ in range(4)]
    q, k, v, dy = (jl.colmajor(t.narrow(1, start, width).clone()) for t in full)
    if rank != 0:
        del full
    out = {}

    def step():
        y, stats, k_ext, v_ext = par.band_attention_fwd(0, q, k, v, ws)
        out["r"] = (y,) + tuple(par.band_attention_bwd(0, q, k, v, y, dy, stats, k_ext, v_ext, ws))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        step()
    barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        a.record(); step(); b.record()          # >= 67 MB per tensor and rank: larger than what stays in L2 between uses
    barrier()
    total = torch.tensor([sum(a.elapsed_time(b) for a, b in evs) * 1e-3], dtype=torch.float64, device=dev)
    # exchange share: the same step with the exchanges alone (no kernels)
    p = plan.p
    ex_evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    st0 = jl.empty((H, width, q.shape[-1]), torch.float32, dev)
    par.exchange_halos([k, v], p)                                 # untimed: buffers of this size exist afterwards
    par.exchange_halos([q, dy, st0, st0], p)
    barrier()
    for a, b in ex_evs:
        a.record()
        par.exchange_halos([k, v], p)
        par.exchange_halos([q, dy, st0, st0], p)
        b.record()
    barrier()
    ex_total = torch.tensor([sum(a.elapsed_time(b) for a, b in ex_evs) * 1e-3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
        dist.all_reduce(ex_total, op=dist.ReduceOp.MAX)
    res = None
    if rank == 0:
        t = float(total.item()) / steps
        cols = sorted({0, p - 1, p, width // 2, width - p - 1, width - 1})
        rows_ = [0, 5, H // 2, H - 1]
        pixels = [h + H * (start + w) for w in cols for h in rows_]
        local = [h + H * w for w in cols for h in rows_]
        err = 0.0
        for unit in (0, nh - 1):
            want = sampled_reference(torch, *full, ws, pixels, unit)
            for got_t, want_t in zip(out["r"], want):
                got = jl.reshape(got_t, (H * width, got_t.shape[-2], got_t.shape[-1]))[local, :, unit].double()
                err = max(err, float((got - want_t).abs().max() / want_t.abs().max()))
        res = {"workload": "one 1024x1024x128 image, ws=21, 8 heads, Dot, flash mode, band split over columns with "
                           "halo exchange, fwd+bwd", "scaling": "strong", "steps": steps, "ms_per_step": t * 1e3,
               "px_per_s": H * W / t, "band_columns": width, "halo_columns": p,
               "exchange_ms_per_step": float(ex_total.item()) / steps * 1e3,
               "exchange_share": float(ex_total.item()) / float(total.item()),
               "parity": {"against": "float64 torch restatement at 24 pixels x 2 units of rank 0's band "
                                     "(band borders and the wrap columns included): y, dq, dk, dv",
                          "max_rel_err": err, "bar": 1e-5, "ok": bool(err < 1e-5)}}
    del out, q, k, v, dy
    ca.ops.release_scratch()
    torch.cuda.empty_cache()
    return res


def units_c5(ca, torch, dist, dev, world, rank, steps):
    """All of BASELINE config 5 (1024 x 1024 x 128, B = 16, ws 21, 8 heads = 128 independent units) sharded
    over batch x heads units with no collective.  A rank walks through its units 16 at a time; the chunks
    reuse one set of buffers (synthetic data: every chunk computes on the same values), which bounds the
    memory to what a 16-unit chunk needs whatever the number of ranks."""
    ops, jl, par = ca.ops, ca.jl, ca.parallel
    H, W, c, ws, units, chunk = 1024, 1024, 16, 21, 128, 16
    _, mine = par.shard_units(units, world, rank)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    q, k, v, dy = (jl.randn(H, W, c, chunk, generator=gen, device=dev) for _ in range(4))
    nchunks = max(1, (mine + chunk - 1) // chunk)

    def step():
        for _ in range(nchunks):
            y, _, stats, fws = ops.attention_fwd(0, 0, q, k, v, ws, False, keep_workspace=True)
            ops.attention_bwd(0, 0, q, k, v, y, dy, stats, ws, fwd_workspace=fws)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    step()
    barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for a, b in evs:
        a.record(); step(); b.record()          # 1 GB per tensor: far larger than L2
    barrier()
    total = torch.tensor([sum(a.elapsed_time(b) for a, b in evs) * 1e-3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
    t = float(total.item()) / steps
    del q, k, v, dy
    ops.release_scratch()
    torch.cuda.empty_cache()
    if rank != 0:
        return None
    return {"workload": "config 5 whole: 1024x1024x128, B=16, ws=21, 8 heads (128 units), Dot, flash mode, fwd+bwd, "
                        "units sharded over ranks, 16 units per launch", "scaling": "strong", "steps": steps,
            "ms_per_step": t * 1e3, "px_per_s": H * W * 16 / t, "units_per_rank": mine}


SLICES = {
    # small cases of the same kernels for profiler captures: name -> a time_config tuple
    "c2": ((128, 96, 64, 2), 15, 4, 0, 0, False, False, "f32"),
    "c2e": ((128, 96, 64, 2), 15, 4, 0, 1, False, False, "f32"),         # the bench shape with entmax: operator chain
    "c2e_sweeps": ((128, 96, 64, 2), 15, 4, 0, 1, False, False, "f32"),  # the same on the scratch-free sweeps
    "c3": ((16384, 64, 4), 127, 8, 1, 1, False, False, "f32"),           # a quarter of config 3's batch (32 units)
    "c3s": ((16384, 64, 4), 127, 8, 1, 0, False, False, "f32"),          # the same with softmax
    "c4": ((320, 320, 32, 2), 7, 1, 0, 0, True, True, "c64"),
    "c5": ((1024, 1024, 32, 1), 21, 2, 0, 0, False, False, "f32"),       # two units of config 5 (0.13 GB per tensor)
    "w7": ((320, 320, 32, 2), 7, 2, 0, 0, False, False, "f32"),          # a 7 x 7 window at 16 channels per head
}


def slice_main(args):
    """Not the headline: a few forward + backward passes of a small slice of a BASELINE configuration (same
    kernels, same window, few units), for profiler captures that must end by themselves.  One JSON line."""
    import torch
    from __graft_entry__ import load_package
    torch.cuda.set_device(0)
    ca = load_package()
    gen = torch.Generator(device="cuda").manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    timed = make_timer(torch, flush)
    if args.slice.endswith("_sweeps"):
        ca.ops.entmax_scratch_limit(0)               # entmax forward: never the A-sized operator chain
    res = time_config(ca, torch, lambda fn: timed(fn, n=3, warm=2), gen, SLICES[args.slice], NOMINAL_FFMA_TFLOPS)
    print(json.dumps({"slice": args.slice, "config": SLICES[args.slice][:5], **res}))


def extra_main(args):
    """Not the headline: the stand-alone operators at the bench shape, one JSON line (L2 flushed before every
    timed call).  The other BASELINE configurations are part of the default run (`other_configs`)."""
    import torch
    from __graft_entry__ import load_package
    torch.cuda.set_device(0)
    ca = load_package()
    ops, jl = ca.ops, ca.jl
    gen = torch.Generator(device="cuda").manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    timed = make_timer(torch, flush)
    out = {"operators_c2_us": {}}
    H, W, C, B, ws, nh = (WORKLOAD[k_] for k_ in ("H", "W", "C", "B", "ws", "nheads"))
    q, k, v = (ca.splitheads(jl.randn(H, W, C, B, generator=gen), nh) for _ in range(3))
    nz = ops.similarity(0, q, k, ws)
    P = ops.row_normalize(nz, (H, W), ws, 0)
    for name, fn in {
        "similarity": lambda: ops.similarity(0, q, k, ws),
        "row_softmax": lambda: ops.row_normalize(nz, (H, W), ws, 0),
        "row_entmax15": lambda: ops.row_normalize(nz, (H, W), ws, 1),
        "row_softmax_bwd": lambda: ops.row_normalize_bwd(P, nz, (H, W), ws, 0),
        "apply": lambda: ops.apply(P, v, ws),
        "apply_transposed": lambda: ops.apply(P, v, ws, True),
        "similarity_bwd": lambda: ops.similarity_bwd(0, q, k, ws, nz),
        "axpby": lambda: ops.axpby(1.0, P, 2.0, nz),
        "sum_rows": lambda: ops.sum_rows(P, (H, W), ws),
        "sum_cols": lambda: ops.sum_cols(P, (H, W), ws),
        "structure": lambda: ops.structure((H, W), ws, (nh, B), "cuda"),
    }.items():
        out["operators_c2_us"][name] = timed(fn) * 1e6
    out["operators_c2_nz_mbytes"] = nz.numel() * 4 / 1e6
    print(json.dumps(out))


# --------------------------------------------------------------------------- B200 arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--extra", nargs="?", const="operators", default=None, choices=["operators"],
                    help="time the stand-alone operators at the bench shape instead of the headline step")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the other BASELINE configurations and the "
                    "sharded config-5 runs (they add a few seconds)")
    ap.add_argument("--no-graph", action="store_true", help="run the end-to-end step eagerly instead of replaying "
                    "its CUDA graph")
    ap.add_argument("--slice", default=None, choices=sorted(SLICES),
                    help="run a few passes of a small slice of a configuration (for profiler captures) and exit")
    args = ap.parse_args()
    if args.slice:
        return slice_main(args)
    if args.extra:
        return extra_main(args)
    if args.impl == "reference":
        return reference_main(args)

    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ca = load_package()
    lib, ops, jl = ca.lib, ca.ops, ca.jl
    warmup = max(args.warmup, 3)
    steps = args.steps

    wl = WORKLOAD
    H, W, C, B, ws, nheads = (wl[k] for k in ("H", "W", "C", "B", "ws", "nheads"))
    px_per_step = H * W * B
    kind, norm = 0, 0

    # every rank owns one batch of the workload (weak scaling over batch x heads units, no collective)
    host = [torch.from_numpy(np.ascontiguousarray(a.T)).pin_memory() for a in make_inputs(wl, rank)]
    q, k, v, r = (ca.splitheads(t.to(dev).permute(3, 2, 1, 0), nheads) for t in host)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    # One step = ca_attention_fwd + ca_attention_bwd through the C ABI on buffers allocated once (as a
    # training loop would keep them): the host does nothing per step but the two calls, so the device
    # never waits for it even when eight ranks share the host's cores.
    m_ = ops.meta_of(q, ws)
    d_ = m_.desc(similarity=kind, normalizer=norm, scale=1.0 / np.sqrt(m_.channels))
    y_ = jl.empty(q.shape, q.dtype, dev)
    stats_ = jl.empty((m_.Np, m_.units), torch.float32, dev)
    grads_ = [jl.empty(q.shape, q.dtype, dev) for _ in range(3)]
    wsf_ = torch.empty(max(lib.ca_attention_fwd_workspace(d_, 0), 16), dtype=torch.uint8, device=dev)
    wsb_ = torch.empty(max(lib.ca_attention_bwd_workspace(d_, 0), 16), dtype=torch.uint8, device=dev)
    ptr_, check_ = ca.ops.ptr, ca._lib.check
    fwd_args = (d_, ptr_(q), ptr_(k), ptr_(v), ptr_(y_), None, ptr_(stats_), ptr_(wsf_))
    bwd_args = (d_, ptr_(q), ptr_(k), ptr_(v), ptr_(y_), ptr_(r), ptr_(stats_), None, None,
                ptr_(grads_[0]), ptr_(grads_[1]), ptr_(grads_[2]), ptr_(wsb_), ptr_(wsf_))

    def step():
        st_ = torch.cuda.current_stream().cuda_stream
        check_(lib.ca_attention_fwd(*fwd_args, st_))
        check_(lib.ca_attention_bwd(*bwd_args, st_))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # clock sampling runs from here to the end of the device work (timed steps, per-kernel timing
    # loops, variants, end-to-end loop); wait for its first line so the timed steps are covered
    sampler = ClockSampler(local)
    sampler.start()
    n0 = lib.ca_probe_launch_count()
    for _ in range(warmup):
        step()
    launches = (lib.ca_probe_launch_count() - n0) // warmup
    sampler.wait_first_sample()
    barrier()
    # the two calls recorded once into a CUDA graph: a replay launches the same five kernels (and the fork and
    # join of the backward's helper stream) without the host between them; a failed capture keeps the plain calls
    step_graph = None
    if not args.no_graph:
        try:
            step_graph, _ = ca.capture(step, warmup=0)
            run_step = step_graph.replay
        except Exception:                                   # noqa: BLE001
            step_graph, run_step = None, step
    else:
        run_step = step
    for _ in range(2):
        run_step()
    barrier()

    # ---- timed region: K steps, each bracketed by CUDA events on the launching stream;
    # L2 (126 MB) is flushed between steps because the 25 MB working set would stay resident.
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    barrier()
    for a, b in ev:
        flush.fill_(1)
        a.record()
        run_step()
        b.record()
    barrier()
    t_steps = [a.elapsed_time(b) * 1e-3 for a, b in ev]
    total = torch.tensor([sum(t_steps)], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(total, op=dist.ReduceOp.MAX)
    total = float(total.item())
    value = px_per_step * steps * world / total

    # ---- per-kernel durations (same inputs, L2 flushed before each launch) for the roofline
    def time_stage(fn, n=20):
        for _ in range(3):
            fn()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in evs:
            flush.fill_(1)
            a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ts = sorted(a.elapsed_time(b) * 1e-3 for a, b in evs)
        return sum(ts) / len(ts), ts[len(ts) // 2]

    y, _, stats = ops.attention_fwd(kind, norm, q, k, v, ws, False)
    m = ops.meta_of(q, ws)
    d = m.desc(similarity=kind, normalizer=norm, scale=1.0 / np.sqrt(m.channels))
    D = torch.empty(m.Np * m.units, dtype=torch.float32, device=dev)
    sws = torch.empty(max(lib.ca_attention_bwd_stage_workspace(d), 16), dtype=torch.uint8, device=dev)
    dq, dk, dv = (jl.empty(q.shape, q.dtype, dev) for _ in range(3))
    st = lambda: torch.cuda.current_stream().cuda_stream
    P = ca.ops.ptr
    stages = {
        "fwd": lambda: ops.attention_fwd(kind, norm, q, k, v, ws, False),
        "bwd_pre": lambda: lib.ca_attention_bwd_pre(d, P(q), P(k), P(v), P(y), P(r), P(stats), None, None, P(D), st()),
        "bwd_dq": lambda: lib.ca_attention_bwd_dq(d, P(q), P(k), P(v), P(r), P(stats), P(D), None, P(dq), P(sws), st()),
        "bwd_dkdv": lambda: lib.ca_attention_bwd_dkdv(d, P(q), P(k), P(v), P(r), P(stats), P(D), None, P(dk), P(dv), P(sws), st()),
    }
    stage_s = {name: time_stage(fn)[0] for name, fn in stages.items()}

    # ---- other configurations of the same shape (not the headline): A materialised, Distance, forward only
    def time_variant(kind_v, want_nz):
        def fn():
            yv, nzv, stv = ops.attention_fwd(kind_v, norm, q, k, v, ws, want_nz)
            ops.attention_bwd(kind_v, norm, q, k, v, yv, r, stv, ws)
        return px_per_step / time_stage(fn, n=10)[0]
    variants = {
        "with_A_px_per_s": time_variant(0, True),
        "distance_px_per_s": time_variant(1, False),
        "fwd_only_px_per_s": px_per_step / stage_s["fwd"],
    }

    # ---- FP32 FMA peak measured on this GPU (not in MEASURED_PEAKS.json)
    sink = torch.empty(148 * 8 * 256, dtype=torch.float32, device=dev)
    ffma_s, _ = time_stage(lambda: lib.ca_probe_ffma(148 * 8, 4096, P(sink), st()), n=10)
    ffma_tflops = 148 * 8 * 256 * 4096 * 16 * 2 * 2 / ffma_s / 1e12

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    dom = max(("fwd", "bwd_dq", "bwd_dkdv"), key=lambda s: stage_s[s])
    traffic = None
    try:   # DRAM bytes per launch of each kernel, from the committed ncu capture of this command
        traffic = json.load(open(os.path.join(ROOT, "profiles", "dram_traffic.json"))).get(dom)
    except (OSError, ValueError):
        pass
    fl, by = algorithmic(wl, dom)
    achieved = fl * px_per_step / stage_s[dom] / 1e12
    fl_all, by_all = algorithmic(wl, "fwd+bwd")
    roofline = {
        "bound": "ffma", "kernel": dom, "achieved": achieved, "peak": ffma_tflops, "unit": "TFLOP/s",
        "frac": achieved / ffma_tflops, "traffic": traffic,
        "peak_source": "FP32 FMA peak measured live by ca_probe_ffma (fma.rn.f32x2, 16 chains/thread); "
                       f"nominal {NOMINAL_FFMA_TFLOPS:.2f}",
        "hbm": {"achieved_gbs": by * px_per_step / stage_s[dom] / 1e9, "peak_gbs": hbm_peak,
                "peak_source": "MEASURED_PEAKS.json" if peaks else "fallback"},
        "step": {"achieved": fl_all * px_per_step / (total / steps) / 1e12,
                 "frac": fl_all * px_per_step / (total / steps) / 1e12 / ffma_tflops,
                 "roofline_px_per_s": ffma_tflops * 1e12 / fl_all},
        "stage_us": {k_: v_ * 1e6 for k_, v_ in stage_s.items()},
    }

    # ---- end to end through the public API: every step copies its inputs from pinned host memory (one
    # staging buffer, one copy), runs circulant_mh_attention + backward, and copies the three gradients and
    # the loss back (one buffer, one copy).  Copy-in, compute and copy-out run on their own streams, double
    # buffered, so that the copies of neighbouring steps overlap the compute (a training loop would prefetch
    # the same way).
    shape_t = tuple(host[0].shape)                     # torch shape (B, C, W, H) = the Julia (H, W, C, B) bytes
    n_el = host[0].numel()
    host_in = torch.empty((4,) + shape_t, dtype=torch.float32).pin_memory()
    for i_, t_ in enumerate(host):
        host_in[i_].copy_(t_)
    host_out = torch.empty(3 * n_el + 1, dtype=torch.float32).pin_memory()
    n_e2e = max(5, min(steps, 30))
    NSLOT = 3                           # buffer slots: the host waits for the copy-out of step i - 3 only
    s_in, s_cmp, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    dev_in = [torch.empty_like(host_in, device=dev) for _ in range(NSLOT)]
    dev_out = [torch.empty(3 * n_el + 1, dtype=torch.float32, device=dev) for _ in range(NSLOT)]
    ev_in = [torch.cuda.Event() for _ in range(NSLOT)]
    ev_cmp = [torch.cuda.Event() for _ in range(NSLOT)]
    ev_out = [torch.cuda.Event() for _ in range(NSLOT)]
    keep = [None] * NSLOT                 # tensors of a slot stay referenced until its copies have finished
    host_busy = [0.0]                   # host time spent enqueueing (waits for the device excluded)
    losses = []
    # per slot, made once: the Julia-shaped views of the staging buffer (q, k, v as leaves that require a
    # gradient, the loss weights) and the views of the output buffer the gradients and the loss are written to
    slot_in, slot_out = [], []
    for s_ in range(NSLOT):
        views = [t.permute(3, 2, 1, 0) for t in dev_in[s_]]
        slot_in.append([v_.detach().requires_grad_(True) for v_ in views[:3]] + [views[3]])
        slot_out.append([dev_out[s_][j_ * n_el:(j_ + 1) * n_el].view(shape_t).permute(3, 2, 1, 0) for j_ in range(3)]
                        + [dev_out[s_][3 * n_el:]])

    def compute(slot):
        """The step itself through the public API: forward, loss, backward, results into the slot's output buffer."""
        qd, kd, vd, rd = slot_in[slot]
        qd.grad = kd.grad = vd.grad = None
        yy, _ = ca.circulant_mh_attention(ca.DotSimilarity(), qd, kd, vd, ws, nheads, return_A=False)
        loss = (yy * rd).sum()
        loss.backward()
        for dst_, t in zip(slot_out[slot], (qd, kd, vd)):
            dst_.copy_(t.grad)
        slot_out[slot][3].copy_(loss.detach().reshape(1))
        return yy, loss

    graphs = [None] * NSLOT               # per slot: the step recorded into a CUDA graph (ca.capture)

    def e2e_step(i):
        slot = i % NSLOT
        ev_out[slot].synchronize()      # the slot's previous outputs have left the device
        losses.append(float(host_out[-1]))
        t_h = time.perf_counter()
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[slot])                    # its previous inputs are no longer read
            dev_in[slot].copy_(host_in, non_blocking=True)
            ev_in[slot].record(s_in)
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(ev_in[slot])
            s_cmp.wait_event(ev_out[slot])                   # dev_out[slot] has been copied out
            if graphs[slot] is not None:
                graphs[slot].replay()
            else:
                keep[slot] = compute(slot) + tuple(slot_in[slot])
            ev_cmp[slot].record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[slot])
            host_out.copy_(dev_out[slot], non_blocking=True)
            ev_out[slot].record(s_out)
        host_busy[0] += time.perf_counter() - t_h

    for i in range(NSLOT + 1):
        e2e_step(i)
    barrier()
    # the step is launch- and host-bound (five kernels of ~50 us behind ~0.6 ms of Python and autograd), so it is
    # recorded once per slot into a CUDA graph and replayed; a failed capture leaves the eager step in place
    graph_note = None
    if not args.no_graph:
        try:
            for slot_ in range(NSLOT):
                graphs[slot_], kept = ca.capture(lambda s_=slot_: compute(s_), stream=s_cmp, warmup=0)
                keep[slot_] = kept + tuple(slot_in[slot_])
        except Exception as e:                              # noqa: BLE001
            graphs = [None] * NSLOT
            graph_note = f"{type(e).__name__}: {e}"[:200]
        barrier()
        for i in range(NSLOT):
            e2e_step(3 + i)
        barrier()
    host_busy[0] = 0.0
    t0 = time.perf_counter()
    for i in range(n_e2e):
        e2e_step(2 * NSLOT + 1 + i)
    barrier()
    e2e_wall = time.perf_counter() - t0
    losses.append(float(host_out[-1]))
    assert all(np.isfinite(losses[2:])), "non-finite loss in the end-to-end loop"
    ops.check_status(dev)
    e2e_t = torch.tensor([e2e_wall], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_t, op=dist.ReduceOp.MAX)
    e2e_value = px_per_step * n_e2e * world / float(e2e_t.item())
    # the link alone: the same bytes in and out per step, both directions at once, nothing computed
    def link_step():
        with torch.cuda.stream(s_in):
            dev_in[0].copy_(host_in, non_blocking=True)
        with torch.cuda.stream(s_out):
            host_out.copy_(dev_out[0], non_blocking=True)
    for _ in range(3):
        link_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        link_step()
    barrier()
    link_t = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(link_t, op=dist.ReduceOp.MAX)
    link_bound = px_per_step * n_e2e * world / float(link_t.item())
    nbytes = n_el * 4
    clocks = sampler.stop()

    # ---- the other BASELINE configurations (one GPU) and the sharded config-5 runs (every N)
    other, sharded = None, {}
    if not args.no_other_configs:
        del q, k, v, r, y, stats, D, sws, dq, dk, dv, dev_in, dev_out, keep, slot_in, slot_out
        ops.release_scratch()
        torch.cuda.empty_cache()
        timed = make_timer(torch, flush)
        # the headline above stands on its own: a failure in one of the side measurements is recorded in its
        # place instead of costing the whole line (every rank takes the same branch: the failures that can
        # happen here -- memory, an unsupported shape -- are the same on all ranks)
        if world == 1:
            gen = torch.Generator(device=dev).manual_seed(0)
            other = {}
            for name, cfg in OTHER_CONFIGS.items():
                try:
                    other[name] = time_config(ca, torch, timed, gen, cfg, ffma_tflops)
                except Exception as e:                      # noqa: BLE001
                    other[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                    torch.cuda.empty_cache()
        for name, fn, n_ in (("units_c5", units_c5, 2), ("band_c5", band_c5, 3)):
            try:
                sharded[name] = fn(ca, torch, dist, dev, world, rank, n_)
            except Exception as e:                          # noqa: BLE001
                sharded[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
                torch.cuda.empty_cache()

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cv, cdt, threads = run_cpu(wl, 5, 1)
        cpu_baseline = {"value": cv, "unit": UNIT, "cores": threads, "kind": "port",
                        "sample": "5 full steps (24576 query pixels each) of the C + OpenMP float32 restatement, "
                                  "work shared as (unit, 256-pixel block) items over all threads; "
                                  "the reference has no CPU path"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": total / steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic (numpy default_rng(rank) standard normal, random weights for the loss)",
            "config": {"workload": "circulant_mh_attention fwd+bwd, H,W,C,B=128,96,64,2 per GPU, ws=15, 4 heads, Dot, "
                                   "softmax, flash mode (A not written)", **wl, "units_per_gpu": nheads * B,
                       "l2": "256 MB buffer written between timed steps (inputs are smaller than L2)",
                       "sharding": "batch x heads units per rank, no collective",
                       "step_launch": ("CUDA graph replay of ca_attention_fwd + ca_attention_bwd (recorded once)"
                                       if step_graph is not None else "two C-ABI calls per step")},
            "roofline": roofline, "cpu_baseline": cpu_baseline, "variants": variants,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 3 * nbytes + 4,
                    "steps": n_e2e, "link_bound_px_per_s": link_bound, "frac_of_link_bound": e2e_value / link_bound,
                    "link_gbs_h2d": 4 * nbytes * n_e2e * world / float(link_t.item()) / 1e9,
                    "host_enqueue_ms_per_step": host_busy[0] / n_e2e * 1e3,
                    "cuda_graph": graphs[0] is not None, **({"cuda_graph_error": graph_note} if graph_note else {}),
                    "timing": "wall clock around the steps, synchronised on both sides, max over ranks; one pinned "
                              "staging buffer and one copy per direction per step; copy-in, compute and copy-out of "
                              "neighbouring steps overlap on three streams; the compute of a step "
                              "(circulant_mh_attention + backward through the public API) is recorded once per "
                              "buffer slot into a CUDA graph (ca.capture) and replayed when cuda_graph is true; "
                              "link_bound = the same copies with nothing computed"},
            "other_configs": other, **sharded,
            "gpu_launches": int(launches), "clocks": clocks,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
