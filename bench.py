#!/usr/bin/env python
"""Benchmark of the W8A8 linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

Prints ONE JSON line (rank 0). See DESIGN.md for what each key means and how the roofline
figures are derived.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

MEASURED_PEAKS = ROOT / "MEASURED_PEAKS.json"
FALLBACK_HBM_GBS = 6650.0


# ------------------------------------------------------------------------------------------
def peaks():
    if MEASURED_PEAKS.exists():
        d = json.loads(MEASURED_PEAKS.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "source": "fallback"}


def algorithmic_bytes(M, N, K, g):
    """int8 weights + fp16 weight scales + fp16 activations in + fp16 out; intermediates count zero."""
    G = (K + g - 1) // g
    return N * K + 2 * N * G + 2 * M * K + 2 * M * N


class ClockSampler:
    """nvidia-smi sampled every 50 ms while the timed regions run."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-i", str(self.gpu), "-lms", "50"], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is not None:
            self.p.terminate()
            try:
                self.p.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.f.name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
ONLY = None  # set from --only


def sweep_cases():
    """configs[1]: the four slow-AR projections x group size {256, 64} x M {1, 4, 16}; M outermost so
    that a weight matrix is not touched again until ~200 MB of other weights went by."""
    from fish_audio_cpp_b200 import synth

    cases = []
    for M in (1, 4, 16):
        for g in (256, 64):
            for name, (K, N) in synth.PROJECTIONS.items():
                if ONLY is None or ONLY == (name, M, g):
                    cases.append({"name": name, "M": M, "N": N, "K": K, "g": g})
    return cases


class DecodeSweep:
    """Device state for configs[1].

    Every weight set exists in several copies (>= 320 MB per set in rotation, far beyond the
    126 MB L2), so no launch finds its weights in cache. One step = one pass over the 24 cases,
    replayed from a CUDA graph (the launches are ~5 us each; launching them one by one from
    Python would measure the interpreter).
    """

    ROTATION_BYTES = 320e6

    def __init__(self, torch, ctx, seed=1234, reference=False, pack=True):
        from fish_audio_cpp_b200 import synth

        self.torch, self.ctx, self.reference = torch, ctx, reference
        self.cases = sweep_cases()
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed)
        rng = np.random.default_rng(seed)
        self.weights = {}
        for g in (256, 64):
            for name, (K, N) in synth.PROJECTIONS.items():
                G = synth.num_groups(K, g)
                copies = max(3, int(np.ceil(self.ROTATION_BYTES / (N * K))))
                self.weights[(name, g)] = [
                    (torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=gen),
                     torch.empty((N, G), dtype=torch.float32, device="cuda").uniform_(1e-3, 5e-3, generator=gen).half())
                    for _ in range(copies)]
                if not reference and pack:
                    # what a loader does once per weight: pack for the decode kernel and register the pair
                    self.packed = getattr(self, "packed", [])
                    for (W, S) in self.weights[(name, g)]:
                        P = torch.empty((ctx.packed_weight_bytes(N, K, g),), dtype=torch.uint8, device="cuda")
                        ctx.pack_weight(W, S, N, K, g, P)
                        ctx.register_packed_weight(W, P)
                        self.packed.append(P)
        self.host_x, self.dev_x, self.dev_y, self.host_y = [], [], [], []
        for c in self.cases:
            x = synth.activations(rng, c["M"], c["K"])
            hx = torch.from_numpy(x).pin_memory()
            self.host_x.append(hx)
            self.dev_x.append(hx.cuda())
            self.dev_y.append(torch.empty((c["M"], c["N"]), dtype=torch.float16, device="cuda"))
            self.host_y.append(torch.empty((c["M"], c["N"]), dtype=torch.float16).pin_memory())
        self.bytes_per_step = sum(algorithmic_bytes(c["M"], c["N"], c["K"], c["g"]) for c in self.cases)
        self.ops_per_step = sum(2 * c["M"] * c["N"] * c["K"] for c in self.cases)
        self.launches_per_step = 2 * len(self.cases) if not reference else sum(
            2 if c["M"] <= 4 else 2 * ((c["K"] + c["g"] - 1) // c["g"]) + 3 for c in self.cases)
        self.h2d = sum(h.numel() * 2 for h in self.host_x)
        self.d2h = sum(h.numel() * 2 for h in self.host_y)
        self.step_no = 0
        self.eager = False
        self.split_k = 0
        self.graphs = {}
        if reference:
            from oracle import fishref

            self.fishref = fishref

    def launch_case(self, i, copy):
        c = self.cases[i]
        W, S = self.weights[(c["name"], c["g"])][copy % len(self.weights[(c["name"], c["g"])])]
        if self.reference:
            s = self.torch.cuda.current_stream().cuda_stream or None
            self.fishref.int8_dequant_gemm_fp16(W.data_ptr(), S.data_ptr(), c["g"], None, None,
                                                self.dev_x[i].data_ptr(), self.dev_y[i].data_ptr(), c["N"], c["M"],
                                                c["K"], s)
        else:
            self.ctx.linear(W, S, c["g"], self.dev_x[i], self.dev_y[i], c["M"], c["N"], c["K"], split_k=self.split_k)

    def one_pass(self, parity, e2e):
        for i, c in enumerate(self.cases):
            if e2e:
                self.dev_x[i].copy_(self.host_x[i], non_blocking=True)
            self.launch_case(i, parity * 3 + (i // 8 if len(self.cases) == 24 else self.step_no))
            if e2e:
                self.host_y[i].copy_(self.dev_y[i], non_blocking=True)

    def graph(self, key, body):
        """Captures body() once and returns the replayable graph (the reference arm runs eagerly:
        its entry point allocates and is not capturable)."""
        t = self.torch
        if key not in self.graphs:
            body()  # eager first: sets kernel attributes, grows nothing afterwards
            t.cuda.synchronize()
            gr = t.cuda.CUDAGraph()
            with t.cuda.graph(gr):
                body()
            self.graphs[key] = gr
        return self.graphs[key]

    def step(self, e2e=False):
        parity = self.step_no % 2
        self.step_no += 1
        if self.reference or self.eager:
            self.one_pass(parity, e2e)
        else:
            self.graph(("pass", parity, e2e), lambda: self.one_pass(parity, e2e)).replay()
        if e2e:
            self.torch.cuda.current_stream().synchronize()

    def per_case(self, min_ms=3.0):
        """Each case alone: one graph of `copies` launches (every copy once), replayed until min_ms."""
        t = self.torch
        out = []
        for i, c in enumerate(self.cases):
            copies = len(self.weights[(c["name"], c["g"])])
            body = lambda: [self.launch_case(i, k) for k in range(copies)]  # noqa: E731
            run = (lambda: body()) if self.reference else self.graph(("case", i), body).replay
            for _ in range(3):
                run()
            t.cuda.synchronize()
            reps, ms = 1, 0.0
            while True:
                e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    run()
                e1.record()
                t.cuda.synchronize()
                ms = e0.elapsed_time(e1)
                if ms >= min_ms or reps >= 4096:
                    break
                reps *= 4
            us = ms * 1e3 / (reps * copies)
            b = algorithmic_bytes(c["M"], c["N"], c["K"], c["g"])
            out.append({"name": c["name"], "M": c["M"], "g": c["g"], "us": round(us, 2),
                        "gbs": round(b / us / 1e3, 1)})
        return out


def cpu_baseline_sweep(budget_s=20.0):
    """The scalar oracle on the host cores: the four projections at M=16, g=256, all rows, one pass."""
    from fish_audio_cpp_b200 import synth
    from oracle import oracle

    threads = oracle.host_threads()
    rng = np.random.default_rng(99)
    total_bytes, total_s, done = 0, 0.0, []
    for name, (K, N) in synth.PROJECTIONS.items():
        M, g = 16, 256
        X, W, ws = synth.activations(rng, M, K), synth.weights(rng, N, K), synth.weight_scales(rng, N, K // g)
        rows = N
        t = oracle.timed_linear(W, ws, g, X, rows, threads)
        total_s += t
        total_bytes += algorithmic_bytes(M, rows, K, g)
        done.append(name)
        if total_s > budget_s:
            break
    return {"value": total_bytes / total_s / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": f"projections {'+'.join(done)} at M=16 g=256, all rows, one pass ({total_s:.2f} s)"}


# ------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["decode_sweep"], default="decode_sweep")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only", default=None, metavar="NAME:M:G",
                    help="restrict the sweep to one case, e.g. gate_up:16:256 (for profiling)")
    ap.add_argument("--no-detail", action="store_true", help="skip the per-case timings")
    ap.add_argument("--split-k", type=int, default=0, help="force the GEMV's K-slice count (tuning aid)")
    ap.add_argument("--no-pack", action="store_true", help="leave weights row-major (skip the loader-side pack)")
    ap.add_argument("--eager", action="store_true", help="launch kernels one by one instead of replaying a graph")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.only:
        global ONLY
        n, m, g = args.only.split(":")
        ONLY = (n, int(m), int(g))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    import torch

    import __graft_entry__ as ge

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: there is no CPU fallback for the product path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pkg = ge.package()
    reference = args.impl == "reference"
    if reference:
        from oracle import fishref

        if not fishref.available():
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "oracle/_ref/libfishref.so was not built (no reference checkout at build time)"}))
            return
        wl = DecodeSweep(torch, None, reference=True)
    else:
        ctx = pkg.Context(local_rank, 0)
        wl = DecodeSweep(torch, ctx, pack=not args.no_pack)

    wl.eager = args.eager
    wl.split_k = args.split_k

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        wl.step()
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        wl.step()
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    # end to end: host buffers in, host buffers out, copies inside the timed region
    e2e_ms = None
    if not reference:
        for _ in range(2):
            wl.step(e2e=True)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            wl.step(e2e=True)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    cases = [] if args.no_detail else wl.per_case()
    clocks = sampler.stop()

    times = torch.tensor([dev_ms, e2e_ms or 0.0], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms_max = times.tolist()
    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    pk = peaks()
    ms_per_step = dev_ms / args.steps
    total_bytes = wl.bytes_per_step * world
    value = total_bytes / (ms_per_step * 1e-3) / 1e9
    per_launch_bytes = wl.bytes_per_step / len(wl.cases)
    per_launch_s = ms_per_step * 1e-3 / len(wl.cases)
    achieved = per_launch_bytes / per_launch_s / 1e9
    line = {
        "metric": "w8a8_decode_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": "configs[1]: slow-AR projections qkv/o/gate_up/down x g{256,64} x M{1,4,16}, "
                               "one W8A8 linear each per step", "cases_per_step": len(wl.cases),
                   "l2": "inputs larger than L2: >= 320 MB of copies per weight set in rotation, M outermost",
                   "parallelism": f"replicas x{world}" if world > 1 else "single GPU",
                   "tops": round(wl.ops_per_step * world / (ms_per_step * 1e-3) / 1e12, 2)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "traffic": None, "peak_source": pk["source"],
                     "kernel": "gemv_kernel" if not reference else "reference kernels",
                     "algorithmic_bytes_per_launch": int(per_launch_bytes)},
        "clocks": clocks,
        "gpu_launches": wl.launches_per_step * args.steps,
        "cases": [dict(c, frac=round(c["gbs"] / pk["hbm_gbs"], 3)) for c in cases],
    }
    if reference:
        line["impl"] = "reference"
        line["cpu_baseline"] = {"value": line["value"], "unit": "GB/s", "cores": 0, "kind": "reference",
                                "sample": "the reference's own CUDA kernels rebuilt for sm_100, stock entry point, "
                                          "on the GPU (the reference has no CPU implementation of this path)"}
        line["e2e"] = {"value": line["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    else:
        e2e_value = total_bytes / (e2e_ms_max / args.steps * 1e-3) / 1e9
        line["e2e"] = {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": wl.h2d,
                       "d2h_bytes_per_step": wl.d2h}
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sweep()
    print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
