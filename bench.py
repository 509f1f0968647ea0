#!/usr/bin/env python
"""Benchmark of the W8A8 linear path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload ...]

Prints ONE JSON line (rank 0): the headline metric of the chosen workload, its roofline figure, the
end-to-end figure with host buffers, the CPU baseline and the clocks seen while it ran.
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


# DRAM traffic / algorithmic bytes of the dominant kernels, from one ncu capture each (dram__bytes_read.sum +
# dram__bytes_write.sum of a launch, summaries under profiles/): gemv_packed_kernel on gate_up M=1 g=256 moved
# 50.249 MB against 50.241 MB; gemm_i8_kernel on gate_up M=2048 g=256 moved 91.8 MB against 135.2 MB (weights,
# scales, codes and activation scales in: 55.7 MB read for 55.5; fp16 out: 36.2 MB of the 79.7 MB had been written
# back when the kernel ended, the rest was still in L2).
# Traffic of both grows in proportion to the bytes a launch touches, so a launch's traffic is that ratio times
# its own algorithmic bytes.
GEMV_TRAFFIC_RATIO = 50.249 / 50.241
GEMM_TRAFFIC_RATIO = 91.8 / 135.2


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
            for name in synth.LAYER_PROJECTIONS:
                K, N = synth.PROJECTIONS[name]
                if ONLY is None or ONLY == (name, M, g):
                    cases.append({"name": name, "M": M, "N": N, "K": K, "g": g})
    return cases


def config0_cases():
    """configs[0]: the single gate-projection GEMM, M = 16, K = 2560, N = 9728, g = 256."""
    from fish_audio_cpp_b200 import synth

    K, N = synth.PROJECTIONS["gate"]
    return [{"name": "gate", "M": 16, "N": N, "K": K, "g": 256}]


class DecodeSweep:
    """Device state for configs[1].

    Every weight set exists in several copies (>= 320 MB per set in rotation, far beyond the
    126 MB L2), so no launch finds its weights in cache. One step = one pass over the 24 cases,
    replayed from a CUDA graph (the launches are ~5 us each; launching them one by one from
    Python would measure the interpreter).
    """

    ROTATION_BYTES = 320e6

    def __init__(self, torch, ctx, seed=1234, reference=False, pack=True, cases=None):
        from fish_audio_cpp_b200 import synth

        self.torch, self.ctx, self.reference = torch, ctx, reference
        self.cases = sweep_cases() if cases is None else cases
        gen = torch.Generator(device="cuda")
        gen.manual_seed(seed)
        rng = np.random.default_rng(seed)
        self.weights = {}
        self.packed = []
        for g in (256, 64):
            for name, (K, N) in synth.PROJECTIONS.items():
                if not any(c["name"] == name and c["g"] == g for c in self.cases):
                    continue
                G = synth.num_groups(K, g)
                copies = max(3, int(np.ceil(self.ROTATION_BYTES / (N * K))))
                self.weights[(name, g)] = [
                    (torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=gen),
                     torch.empty((N, G), dtype=torch.float32, device="cuda").uniform_(1e-3, 5e-3, generator=gen).half())
                    for _ in range(copies)]
                if not reference and pack:
                    # what a loader does once per weight: pack for the decode kernel and register the pair
                    for (W, S) in self.weights[(name, g)]:
                        P = torch.empty((ctx.packed_weight_bytes(N, K, g),), dtype=torch.uint8, device="cuda")
                        ctx.pack_weight(W, S, N, K, g, P)
                        ctx.register_packed_weight(W, P, N, K, g)
                        self.packed.append((W, P))
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

    def close(self):
        """Unregisters the packed images (before the tensors are freed) and drops the graphs."""
        for W, _ in self.packed:
            self.ctx.register_packed_weight(W, None)
        self.packed, self.graphs = [], {}

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


class PrefillSweep:
    """configs[2]: the four projections x g{256,64} x M{2048,8192}, one W8A8 linear each (row quantiser +
    tcgen05 GEMM), fp16 in, fp16 out. Activations + weights of a case (up to ~370 MB) exceed L2 together
    with the rotation over the eight weight sets."""

    def __init__(self, torch, ctx, seed=4321, Ms=(2048, 8192), reference=False):
        from fish_audio_cpp_b200 import synth

        self.torch, self.ctx, self.reference = torch, ctx, reference
        if reference:
            from oracle import fishref

            self.fishref = fishref
        proj = {n: synth.PROJECTIONS[n] for n in synth.LAYER_PROJECTIONS}
        gen = torch.Generator(device="cuda").manual_seed(seed)
        self.cases, self.w = [], {}
        for g in (256, 64):
            for name, (K, N) in proj.items():
                G = K // g
                self.w[(name, g)] = (
                    torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda", generator=gen),
                    torch.empty((N, G), dtype=torch.float32, device="cuda").uniform_(1e-3, 5e-3, generator=gen).half())
        self.x = {}
        for M in Ms:
            for K in sorted({k for k, _ in proj.values()}):
                x = torch.randn((M, K), dtype=torch.float32, device="cuda", generator=gen)
                idx = torch.randperm(K, device="cuda", generator=gen)[:max(1, round(0.005 * K))]
                x[:, idx] *= 20.0
                self.x[(M, K)] = x.half()
        for M in Ms:
            for g in (256, 64):
                for name, (K, N) in proj.items():
                    if ONLY is None or ONLY == (name, M, g):
                        self.cases.append({"name": name, "M": M, "N": N, "K": K, "g": g})
        self.y = torch.empty((max(Ms), 19456), dtype=torch.float16, device="cuda")
        self.ops_per_step = sum(2 * c["M"] * c["N"] * c["K"] for c in self.cases)
        self.bytes_per_step = sum(algorithmic_bytes(c["M"], c["N"], c["K"], c["g"]) for c in self.cases)
        # the reference: quantiser + per group (cuBLAS GEMM + accumulate) + memset + cast (int8_gemm.cu:415-505)
        self.launches_per_step = 2 * len(self.cases) if not reference else sum(
            2 * (c["K"] // c["g"]) + 3 for c in self.cases)
        self.eager, self.split_k, self.graphs = False, 0, {}
        self.h2d = self.d2h = 0

    def close(self):
        self.w, self.x, self.y = {}, {}, None

    def run_case(self, c):
        W, S = self.w[(c["name"], c["g"])]
        if self.reference:
            s = self.torch.cuda.current_stream().cuda_stream or None
            self.fishref.int8_dequant_gemm_fp16(W.data_ptr(), S.data_ptr(), c["g"], None, None,
                                                self.x[(c["M"], c["K"])].data_ptr(), self.y.data_ptr(), c["N"], c["M"],
                                                c["K"], s)
        else:
            self.ctx.linear(W, S, c["g"], self.x[(c["M"], c["K"])], self.y, c["M"], c["N"], c["K"])

    def step(self, e2e=False):
        for c in self.cases:
            self.run_case(c)

    def per_case(self, min_ms=20.0):
        t, out = self.torch, []
        for c in self.cases:
            for _ in range(2):
                self.run_case(c)
            t.cuda.synchronize()
            reps = 1
            while True:
                e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    self.run_case(c)
                e1.record()
                t.cuda.synchronize()
                ms = e0.elapsed_time(e1)
                if ms >= min_ms or reps >= 256:
                    break
                reps *= 2
            us = ms * 1e3 / reps
            out.append({"name": c["name"], "M": c["M"], "g": c["g"], "us": round(us, 1),
                        "tops": round(2 * c["M"] * c["N"] * c["K"] / us / 1e6, 1)})
        return out


class DecodeStack:
    """configs[3]: the full slow-AR decoder stack, batch 8, context 1024, g256, tensor-parallel over the
    ranks of the job. One step = one token for each of the 8 sequences, replayed from a CUDA graph.
    reference=True: the same step through the reference's own CUDA kernels (oracle/ref_stack.py), eager, built with
    torch alone (the product library is not loaded)."""

    def __init__(self, torch, ctx, world, rank, dist, layers=36, batch=8, context=1024, group=256, reference=False,
                 tp_mode="fused"):
        from fish_audio_cpp_b200 import stack as S

        self.torch, self.ctx, self.dist, self.world = torch, ctx, dist, world
        cfg = S.SlowARConfig(n_layer=layers, group=group)
        self.cfg, self.batch, self.context = cfg, batch, context
        self.tp_mode = tp_mode if world > 1 else "none"
        self.host_x = (torch.randn((batch, cfg.dim), generator=torch.Generator().manual_seed(3)) * 0.5).half().pin_memory()
        self.dev_x = self.host_x.cuda()
        self.host_out = torch.empty((batch, cfg.dim), dtype=torch.float16).pin_memory()
        self.graphs, self.eager, self.split_k, self.one_launch, self.cases = {}, False, 0, False, []
        self.h2d, self.d2h = self.host_x.numel() * 2, self.host_out.numel() * 2
        self.steps_done = 0
        weight_bytes_full = layers * sum(n * k + 2 * n * (k // group) for n, k in (
            ((cfg.n_head + 2 * cfg.n_kv) * cfg.head_dim, cfg.dim), (cfg.dim, cfg.n_head * cfg.head_dim),
            (2 * cfg.inter, cfg.dim), (cfg.dim, cfg.inter)))
        kv_full = 2 * batch * context * layers * cfg.n_kv * cfg.head_dim * 2
        if reference:
            from oracle import ref_stack

            self.st = None
            self.ref = ref_stack.ReferenceStack(torch, cfg, batch, context, max_new=128, seed=7)
            self.launches_per_step = 0
            self.bytes_per_step = weight_bytes_full + kv_full
            self.ops_per_step = 0
            return
        ar, gather = None, None
        if world > 1 and tp_mode == "nccl":
            ar = lambda t: dist.all_reduce(t)  # noqa: E731  (fp16 sum over NVLink, NCCL: the baseline)
        if world > 1 and tp_mode == "fused":
            def gather(handle):
                out = [None] * world
                dist.all_gather_object(out, handle)
                return out
        self.st = S.SlowARStack(torch, ctx, cfg, batch, context, max_new=128, tp_rank=rank, tp_size=world,
                                seed=7, all_reduce=ar, pack=True, tp_mode=tp_mode, gather_handles=gather)
        self.ref = None
        self.launches_per_step = self.st.launches_per_step
        # algorithmic bytes of one step on one rank: its weight shards + scales, the KV it reads, activations ~0
        self.bytes_per_step = self.st.weight_bytes + self.st.kv_bytes_per_step(context)
        self.ops_per_step = 2 * batch * sum(lw[n].numel() for lw in self.st.layers for n in ("wqkv", "wo", "w13", "w2"))

    def close(self):
        self.graphs = {}
        if self.st is not None:
            self.st.close()

    def body(self, e2e):
        if e2e:
            self.dev_x.copy_(self.host_x, non_blocking=True)
        if self.one_launch:
            self.st.decode_step_one_launch(self.dev_x)
        else:
            self.st.decode_step(self.dev_x)
        if e2e:
            self.host_out.copy_(self.st.out, non_blocking=True)

    def timeline(self):
        """Median microseconds per phase and per barrier of one layer in the last one-launch step (CTA 0's
        device clock; layer 0 left out: its first phase has no residual to add)."""
        t = np.asarray(self.ctx.decode_stack_timeline(self.st.one_launch_descriptor()), dtype=np.int64)
        L = self.cfg.n_layer
        per = np.diff(t)[:18 * L].reshape(L, 18)[1:] if L > 1 else np.diff(t)[:18].reshape(1, 18)
        med = np.median(per, axis=0) / 1e3
        names = ["A norm+quant", "B wqkv", "C rope+kv+attention", "D merge+quant", "E wo", "F norm+quant", "G w13+swiglu",
                 "H quant", "I w2"]
        out = {}
        for i, n in enumerate(names):
            out[n] = round(float(med[2 * i]), 2)
            out[n + " | barrier"] = round(float(med[2 * i + 1]), 2)
        out["layer"] = round(float(med.sum()), 2)
        out["step"] = round(float(t[-1] - t[0]) / 1e3, 1)
        return out

    def time_linears(self, reps=20):
        """(average seconds per launch, algorithmic bytes per launch) of the four linears of every layer,
        replayed alone from a graph: the dominant kernel on its own, timed with CUDA events."""
        t = self.torch
        self.st.linears_only()
        t.cuda.synchronize()
        gr = t.cuda.CUDAGraph()
        with t.cuda.graph(gr):
            self.st.linears_only()
        for _ in range(3):
            gr.replay()
        e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            gr.replay()
        e1.record()
        t.cuda.synchronize()
        launches = 4 * self.cfg.n_layer
        acts = 2 * self.batch * (2 * self.cfg.dim + self.st.attn_k + self.st.inter_l) + \
            2 * self.batch * (self.st.qkv_n + 2 * self.cfg.dim + self.st.inter_l)
        per_launch_bytes = self.st.weight_bytes / launches + acts / 4
        return e0.elapsed_time(e1) * 1e-3 / (reps * launches), per_launch_bytes

    def step(self, e2e=False):
        t = self.torch
        if self.ref is not None:
            self.ref.reset_positions()
            self.ref.decode_step(self.dev_x, advance=False)
            return
        # the context grows by one token per step; go back to 1024 every 64 steps so that it stays "1024"
        if self.steps_done and self.steps_done % 64 == 0:
            self.st.reset_positions()
        self.steps_done += 1
        if self.eager:
            self.body(e2e)
        else:
            key = ("step", e2e)
            if key not in self.graphs:
                self.body(e2e)
                t.cuda.synchronize()
                gr = t.cuda.CUDAGraph()
                with t.cuda.graph(gr):
                    self.body(e2e)
                self.graphs[key] = gr
            self.graphs[key].replay()
        if e2e:
            t.cuda.current_stream().synchronize()

    def per_case(self, min_ms=3.0):
        return []


class FastARFrame:
    """configs[4]: the fast-AR codebook decoder. One step = one frame: 10 codebook steps, each a 4-layer stack
    (hidden 2560, 32q/8kv x128, SwiGLU 9728, no qk-norm, W8A8 g64) at batch 8 over the codebooks decoded so far
    (the mirror of DualAREngine::fast_codebook_decode_device, src/engine/dual_ar_engine.cc:769-844), then the final
    norm and the codebook head 2560 -> 4096 (g64). Sampling and the embedding lookup of the sampled code are left
    out: every codebook step gets the same synthetic input rows. The frame is replayed from one CUDA graph.
    `lm_head()` times the slow AR's int8 LM head 2560 -> 155776 (g256) at M = 1 and 8 on the side.
    reference=True: the same frame through the reference's own CUDA kernels, eager (oracle/ref_stack.py)."""

    def __init__(self, torch, ctx, batch=8, codebooks=10, reference=False):
        from fish_audio_cpp_b200 import stack as S

        self.torch, self.ctx, self.batch, self.codebooks, self.reference = torch, ctx, batch, codebooks, reference
        cfg = S.SlowARConfig(n_layer=4, group=64, qk_norm=False)
        self.cfg = cfg
        gen = torch.Generator(device="cuda").manual_seed(5)
        self.head_w = torch.randint(-127, 128, (4096, cfg.dim), dtype=torch.int8, device="cuda", generator=gen)
        self.head_s = torch.empty((4096, cfg.dim // 64), dtype=torch.float32, device="cuda").uniform_(
            1e-3, 5e-3, generator=gen).half()
        self.logits = torch.empty((batch, 4096), dtype=torch.float16, device="cuda")
        self.host_x = (torch.randn((batch, cfg.dim), generator=torch.Generator().manual_seed(3)) * 0.5).half().pin_memory()
        self.dev_x = self.host_x.cuda()
        self.host_logits = torch.empty((batch, 4096), dtype=torch.float16).pin_memory()
        self.graphs, self.eager, self.split_k, self.cases = {}, False, 0, []
        self.h2d, self.d2h = self.host_x.numel() * 2, self.host_logits.numel() * 2
        head_bytes = self.head_w.numel() + self.head_s.numel() * 2
        kv = sum(2 * batch * (t + 1) * cfg.n_layer * cfg.n_kv * cfg.head_dim * 2 for t in range(codebooks))
        g = cfg.group
        stack_weight_bytes = cfg.n_layer * sum(n * k + 2 * n * (k // g) for n, k in (
            ((cfg.n_head + 2 * cfg.n_kv) * cfg.head_dim, cfg.dim), (cfg.dim, cfg.n_head * cfg.head_dim),
            (2 * cfg.inter, cfg.dim), (cfg.dim, cfg.inter)))
        self.bytes_per_step = codebooks * (stack_weight_bytes + head_bytes) + kv
        if reference:
            from oracle import fishref, ref_stack

            self.fishref = fishref
            self.st = None
            self.ref = ref_stack.ReferenceStack(torch, cfg, batch, 0, max_new=32, seed=17)
            self.launches_per_step = 0
            self.ops_per_step = 0
            return
        self.ref = None
        self.st = S.SlowARStack(torch, ctx, cfg, batch, 0, max_new=32, seed=17)
        P = torch.empty((ctx.packed_weight_bytes(4096, cfg.dim, 64),), dtype=torch.uint8, device="cuda")
        ctx.pack_weight(self.head_w, self.head_s, 4096, cfg.dim, 64, P)
        ctx.register_packed_weight(self.head_w, P, 4096, cfg.dim, 64)
        self._keep = [P]
        self.launches_per_step = codebooks * (self.st.launches_per_step + 2)
        self.ops_per_step = codebooks * 2 * batch * (sum(lw[n].numel() for lw in self.st.layers
                                                           for n in ("wqkv", "wo", "w13", "w2")) + self.head_w.numel())

    def close(self):
        self.graphs = {}
        if self.st is not None:
            self.ctx.register_packed_weight(self.head_w, None)
            self.st.close()

    def body(self, e2e):
        if e2e:
            self.dev_x.copy_(self.host_x, non_blocking=True)
        for _ in range(self.codebooks):
            out = self.st.decode_step(self.dev_x)
            self.ctx.linear(self.head_w, self.head_s, 64, out, self.logits, self.batch, 4096, self.cfg.dim)
        self.st.reset_positions()
        if e2e:
            self.host_logits.copy_(self.logits, non_blocking=True)

    def reference_body(self):
        self.ref.reset_positions()
        for _ in range(self.codebooks):
            out = self.ref.decode_step(self.dev_x)
            self.fishref.int8_dequant_gemm_fp16(self.head_w.data_ptr(), self.head_s.data_ptr(), 64, None, None,
                                                out.data_ptr(), self.logits.data_ptr(), 4096, self.batch, self.cfg.dim)

    def step(self, e2e=False):
        t = self.torch
        if self.reference:
            self.reference_body()
            return
        if self.eager:
            self.body(e2e)
        else:
            if e2e not in self.graphs:
                self.body(e2e)
                t.cuda.synchronize()
                gr = t.cuda.CUDAGraph()
                with t.cuda.graph(gr):
                    self.body(e2e)
                self.graphs[e2e] = gr
            self.graphs[e2e].replay()
        if e2e:
            t.cuda.current_stream().synchronize()

    def per_case(self, min_ms=3.0):
        return []

    def lm_head(self, vocab=155776, reps=20):
        """The slow AR's LM head as an int8 linear (the reference keeps it fp16: tools/quant_utils.py:37-52), M = 1
        and 8, g256, packed: microseconds and GB/s of algorithmic bytes, weights (399 MB) larger than L2."""
        t, ctx, K = self.torch, self.ctx, self.cfg.dim
        gen = t.Generator(device="cuda").manual_seed(9)
        W = t.randint(-127, 128, (vocab, K), dtype=t.int8, device="cuda", generator=gen)
        Sc = t.empty((vocab, K // 256), dtype=t.float32, device="cuda").uniform_(1e-3, 5e-3, generator=gen).half()
        P = t.empty((ctx.packed_weight_bytes(vocab, K, 256),), dtype=t.uint8, device="cuda")
        ctx.pack_weight(W, Sc, vocab, K, 256, P)
        ctx.register_packed_weight(W, P, vocab, K, 256)
        out = {}
        for M in (1, 8):
            X = (t.randn((M, K), device="cuda", generator=gen) * 0.5).half()
            Y = t.empty((M, vocab), dtype=t.float16, device="cuda")
            for _ in range(3):
                ctx.linear(W, Sc, 256, X, Y, M, vocab, K)
            e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(reps):
                ctx.linear(W, Sc, 256, X, Y, M, vocab, K)
            e1.record()
            t.cuda.synchronize()
            us = e0.elapsed_time(e1) * 1e3 / reps
            out[f"M{M}"] = {"us": round(us, 1), "gbs": round(algorithmic_bytes(M, vocab, K, 256) / us / 1e3, 1)}
        ctx.register_packed_weight(W, None)
        # the rows the decode sampler reads (semantic range + end of sequence) as a table of their own
        from fish_audio_cpp_b200 import lm_head as lmh

        rows = lmh.sampled_rows()
        Wc, Scc = lmh.compact_head(W, Sc, rows)
        n = len(rows)
        Pc = t.empty((ctx.packed_weight_bytes(n, K, 256),), dtype=t.uint8, device="cuda")
        ctx.pack_weight(Wc, Scc, n, K, 256, Pc)
        ctx.register_packed_weight(Wc, Pc, n, K, 256)
        flush = t.empty((256 << 20,), dtype=t.uint8, device="cuda")
        for M in (1, 8):
            X = (t.randn((M, K), device="cuda", generator=gen) * 0.5).half()
            Y = t.empty((M, n), dtype=t.float16, device="cuda")
            for _ in range(3):
                ctx.linear(Wc, Scc, 256, X, Y, M, n, K)
            total = 0.0
            for _ in range(reps):  # 10.5 MB of weights would sit in L2: flush it between the timed launches
                flush.fill_(1)
                e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
                e0.record()
                ctx.linear(Wc, Scc, 256, X, Y, M, n, K)
                e1.record()
                t.cuda.synchronize()
                total += e0.elapsed_time(e1) * 1e3
            us = total / reps
            out[f"sampled_rows_M{M}"] = {"rows": n, "us": round(us, 1),
                                         "gbs": round(algorithmic_bytes(M, n, K, 256) / us / 1e3, 1)}
        ctx.register_packed_weight(Wc, None)
        return out


def cpu_baseline_stack(budget_s=12.0):
    """The scalar oracle on the host cores over one decoder layer's four linears at batch 8 (g256), repeated
    until about `budget_s` seconds of CPU work have been timed, scaled to 36 layers: the linears are > 99 % of
    a CPU step, norms/rope/attention are left out of the sample."""
    from fish_audio_cpp_b200 import synth
    from oracle import oracle

    threads = oracle.host_threads()
    rng = np.random.default_rng(99)
    cases = []
    for name in synth.LAYER_PROJECTIONS:
        K, N = synth.PROJECTIONS[name]
        cases.append((synth.activations(rng, 8, K), synth.weights(rng, N, K), synth.weight_scales(rng, N, K // 256), N))
    total_s, reps = 0.0, 0
    while total_s < budget_s and reps < 2000:
        for X, W, ws, N in cases:
            total_s += oracle.timed_linear(W, ws, 256, X, N, threads)
        reps += 1
    per_layer = total_s / reps
    return {"value": 8.0 / (per_layer * 36), "unit": "tokens/s", "cores": threads, "kind": "port",
            "sample": f"the four linears of one layer at batch 8, g256, all rows, {reps} times ({total_s:.1f} s of "
                      f"CPU work, {per_layer * 1e3:.1f} ms per layer), x36 layers"}


def cpu_baseline_sweep(budget_s=20.0):
    """The scalar oracle on the host cores: the four projections at M=16, g=256, all rows, one pass."""
    from fish_audio_cpp_b200 import synth
    from oracle import oracle

    threads = oracle.host_threads()
    rng = np.random.default_rng(99)
    total_bytes, total_s, done = 0, 0.0, []
    for name in synth.LAYER_PROJECTIONS:
        K, N = synth.PROJECTIONS[name]
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


def cpu_baseline_prefill(budget_s=15.0):
    """The scalar oracle on the host cores: a 64-token slice of the gate_up projection at g=256 (all 19456 rows),
    scaled by its ops; reported in TOPS."""
    from fish_audio_cpp_b200 import synth
    from oracle import oracle

    threads = oracle.host_threads()
    rng = np.random.default_rng(98)
    K, N = synth.PROJECTIONS["gate_up"]
    M, g = 64, 256
    X, W, ws = synth.activations(rng, M, K), synth.weights(rng, N, K), synth.weight_scales(rng, N, K // g)
    total_s, reps = 0.0, 0
    while total_s < budget_s and reps < 50:
        total_s += oracle.timed_linear(W, ws, g, X, N, threads)
        reps += 1
    return {"value": 2.0 * M * N * K * reps / total_s / 1e12, "unit": "TOPS", "cores": threads, "kind": "port",
            "sample": f"gate_up at g=256, a {M}-token slice, all rows, {reps} times ({total_s:.1f} s of CPU work)"}


# ------------------------------------------------------------------------------------------
TRACE_KERNELS = {2: "rowquant", 3: "groupquant", 4: "attention", 5: "tp_row", 10: "gemv", 11: "gemv+norm",
                 14: "gemv+rowtail", 18: "gemv+grouptail"}


def read_device_trace():
    """Records left by a diagnostic build of the library (python fish-audio-cpp_b200/build.py --define W8A8_TRACE
    --out DIR, then W8A8_LIBRARY=DIR/libw8a8.so): thread 0 of the first and of the last CTA of every decode kernel
    stamps the GPU's nanosecond timer at kernel entry, after the dependency wait and at the CTA's end. Returns a
    list of tuples (t_entry, t_waited, t_end, kernel id, cta, ctas, aux) and clears the device buffers; [] when the
    loaded library was not built with the trace."""
    import ctypes as C

    from fish_audio_cpp_b200 import capi

    class Rec(C.Structure):
        _fields_ = [("t_entry", C.c_ulonglong), ("t_waited", C.c_ulonglong), ("t_end", C.c_ulonglong),
                    ("id", C.c_uint), ("cta", C.c_uint), ("ctas", C.c_uint), ("aux", C.c_uint)]
    lib, out = capi.load_library(), []
    for name in ("gemv_packed", "quant", "attn", "tp"):
        fn = getattr(lib, "w8a8_trace_read_" + name, None)
        if fn is None:
            return []
        fn.restype = C.c_int
        buf = (Rec * 16384)()
        n = fn(buf, 16384)
        out += [(r.t_entry, r.t_waited, r.t_end, r.id, r.cta, r.ctas, r.aux) for r in buf[:max(n, 0)]]
    return out


def step_timeline(torch, wl):
    """One replayed decode step as a per-kernel device timeline: for every position in a layer's launch sequence the
    median over the layers of (a) the edge: from the end of the kernel before it to the moment its own dependency
    wait returned, and (b) the body: from there to its last recorded CTA's end. Microseconds."""
    read_device_trace()
    wl.step()
    torch.cuda.synchronize()
    recs = sorted(read_device_trace(), key=lambda r: r[2])
    if not recs:
        return {"error": "the loaded library has no trace (build it with --define W8A8_TRACE and set W8A8_LIBRARY)"}
    inst, pending = [], {}
    for r in recs:
        key = (r[3], r[5], r[6])
        if r[5] == 1:
            inst.append(dict(id=r[3], aux=r[6], W=r[1], E=r[2]))
        elif key in pending and pending[key][4] != r[4]:
            o = pending.pop(key)
            inst.append(dict(id=r[3], aux=r[6], W=max(o[1], r[1]), E=max(o[2], r[2])))
        else:
            pending[key] = r
    inst.sort(key=lambda k: k["E"])
    L = wl.cfg.n_layer
    per = len(inst) // L
    if per == 0 or len(inst) < per * L:
        return {"error": f"{len(inst)} kernel instances do not divide into {L} layers"}
    edges, bodies = np.zeros((L - 1, per)), np.zeros((L - 1, per))
    for l in range(1, L):
        for j in range(per):
            k, prev = inst[l * per + j], inst[l * per + j - 1]
            edges[l - 1, j] = (k["W"] - prev["E"]) / 1e3
            bodies[l - 1, j] = (k["E"] - k["W"]) / 1e3
    rows = []
    for j in range(per):
        k = inst[per + j]
        name = TRACE_KERNELS.get(k["id"], str(k["id"])) + (f"[N={k['aux']}]" if k["aux"] else "")
        rows.append([name, round(float(np.median(edges[:, j])), 2), round(float(np.median(bodies[:, j])), 2)])
    out = {"per_layer": rows, "layer_us": round(float(np.median(edges, 0).sum() + np.median(bodies, 0).sum()), 2),
           "columns": ["kernel", "edge_us", "body_us"]}
    import ctypes as C

    from fish_audio_cpp_b200 import capi
    fn = getattr(capi.load_library(), "w8a8_trace_read_attn_phases", None)
    if fn is not None:  # phases of the attention launch of the step's last layer, CTA (0, 0, 0), microseconds from entry
        buf = (C.c_ulonglong * 8)()
        fn.restype = C.c_int
        if fn(buf) == 8:
            names = ["entry", "dependency_wait_returned", "q_and_new_rows_ready", "first_block_in_hand", "blocks_done",
                     "warps_merged", "cluster_synced", "end"]
            out["attention_phases_us"] = {n: round((buf[i] - buf[0]) / 1e3, 2) for i, n in enumerate(names)}
    return out


def gemm_timeline(torch, pkg, M=8192, groups=(256, 64)):
    """Where a tile of the prefill GEMM spends its time (gate_up, M tokens): a diagnostic build of the library
    (--define W8A8_TRACE) stamps the SM clock in CTA 0's MMA-issuing lane and first epilogue warp per K-group and in
    its producer lane per K-block. Medians over four tiles' worth of groups, microseconds at 1965 MHz."""
    import ctypes as C

    from fish_audio_cpp_b200 import capi
    fn = getattr(capi.load_library(), "w8a8_trace_read_gemm", None)
    if fn is None:
        return {"error": "the loaded library has no trace (build it with --define W8A8_TRACE and set W8A8_LIBRARY)"}
    fn.restype, fn.argtypes = C.c_int, [C.c_void_p, C.c_int]
    K, N = 2560, 19456
    ctx = pkg.Context(torch.cuda.current_device(), 0)
    out = {}
    for g in groups:
        G = K // g
        W = torch.randint(-127, 128, (N, K), dtype=torch.int8, device="cuda")
        ws = (torch.rand((N, G), device="cuda") * 4e-3 + 1e-3).half()
        Xq = torch.randint(-127, 128, (M, K), dtype=torch.int8, device="cuda")
        Xs = torch.rand((M, G), device="cuda") * 1e-2 + 1e-3
        Y = torch.empty((M, N), dtype=torch.float16, device="cuda")
        buf = np.zeros((3, 512, 4), np.uint64)
        for _ in range(3):
            ctx.linear_q(W, ws, g, Xq, Xs, Y, M, N, K)
        torch.cuda.synchronize()
        fn(buf.ctypes.data, buf.nbytes)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ctx.linear_q(W, ws, g, Xq, Xs, Y, M, N, K)
        e1.record()
        torch.cuda.synchronize()
        if fn(buf.ctypes.data, buf.nbytes) <= 0:
            return {"error": "reading the trace failed"}
        b = buf.astype(np.int64)
        pro, mma, epi = b[0], b[1], b[2]
        lo, hi = 2 * G, min(6 * G, 500)
        us = lambda x: round(float(np.median(x)) / 1965.0, 3)  # noqa: E731
        kbs = K // 128
        out[f"g{g}"] = {
            "launch_us": round(e0.elapsed_time(e1) * 1e3, 1),
            "mma_lane_per_group": {"wait_operands": us(mma[lo:hi, 1] - mma[lo:hi, 0]), "wait_accumulator_slice": us(mma[lo:hi, 2] - mma[lo:hi, 1]),
                                   "issue_mmas_and_commit": us(mma[lo:hi, 3] - mma[lo:hi, 2]), "period": us(np.diff(mma[lo:hi, 0]))},
            "epilogue_warp_per_group": {"wait_sums": us(epi[lo:hi, 1] - epi[lo:hi, 0]), "load_and_promote_until_release": us(epi[lo:hi, 2] - epi[lo:hi, 1]),
                                        "rest_of_promote": us(epi[lo:hi, 3] - epi[lo:hi, 2]), "period": us(np.diff(epi[lo:hi, 0]))},
            "producer_lane_per_kblock": {"wait_free_stage": us(pro[2 * kbs:min(6 * kbs, 500), 1] - pro[2 * kbs:min(6 * kbs, 500), 0]),
                                         "period": us(np.diff(pro[2 * kbs:min(6 * kbs, 500), 0]))},
            # from the last promote of a tile to the first wait of the next: output conversion, store, scale preload
            "between_tiles": round(float(epi[3 * G, 0] - epi[3 * G - 1, 3]) / 1965.0, 3) if 3 * G < 512 else None,
        }
        del W, ws, Xq, Xs, Y
    ctx.close()
    return out


def int8_library_tops(torch):
    """cuBLASLt int8 -> int32 at 8192^3 through torch._int_mm: the measured int8 tensor figure of this GPU."""
    t = torch
    try:
        a = t.randint(-127, 128, (8192, 8192), dtype=t.int8, device="cuda")
        bm = t.randint(-127, 128, (8192, 8192), dtype=t.int8, device="cuda")
        for _ in range(3):
            t._int_mm(a, bm)
        t.cuda.synchronize()
        best = 1e9
        for _ in range(10):
            e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
            e0.record()
            t._int_mm(a, bm)
            e1.record()
            t.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1))
        return round(2 * 8192 ** 3 / (best * 1e-3) / 1e12, 1)
    except Exception:  # noqa: BLE001
        return None


def int8_peak_tops():
    bf16 = None
    if MEASURED_PEAKS.exists():
        bf16 = float(json.loads(MEASURED_PEAKS.read_text()).get("bf16_tflops", 0)) or None
    return (2 * bf16 if bf16 else 2 * 1590.0), bool(bf16)


def timed_steps(torch, wl, steps, warmup=3):
    for _ in range(warmup):
        wl.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        wl.step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def extra_metrics(torch, ctx, pk):
    """The other headline configurations, measured in the same process after the decode stack's timed region (one
    GPU): the single gate GEMM of configs[0], the decode sweep of configs[1], the prefill GEMMs of configs[2] with the
    library int8 figure, the fast-AR frame of configs[4]. Each with CUDA events over graph replays / repeated launches
    whose weights rotate through more than L2 holds."""
    out = {}
    hbm = pk["hbm_gbs"]
    wl = DecodeSweep(torch, ctx, cases=config0_cases())
    c = wl.per_case()[0]
    out["config0_gate_M16_K2560_N9728_g256"] = {"us": c["us"], "gbs": c["gbs"], "frac_of_hbm": round(c["gbs"] / hbm, 3),
                                                "tops": round(2 * 16 * 9728 * 2560 / c["us"] / 1e6, 1),
                                                "includes": "quantiser launch + linear launch"}
    wl.close()
    del wl
    wl = DecodeSweep(torch, ctx)
    ms = timed_steps(torch, wl, 30)
    cases = wl.per_case()
    worst = min(cases, key=lambda c: c["gbs"])
    best = max(cases, key=lambda c: c["gbs"])
    agg = wl.bytes_per_step / (ms * 1e-3) / 1e9
    out["configs1_decode_sweep"] = {
        "aggregate_gbs": round(agg, 1), "aggregate_frac_of_hbm": round(agg / hbm, 3),
        "worst": dict(worst, frac=round(worst["gbs"] / hbm, 3)), "best": dict(best, frac=round(best["gbs"] / hbm, 3)),
        "frac_by_M": {str(M): round(float(np.mean([c["gbs"] for c in cases if c["M"] == M])) / hbm, 3) for M in (1, 4, 16)},
        "cases": [[c["name"], c["M"], c["g"], c["us"], round(c["gbs"] / hbm, 3)] for c in cases]}
    wl.close()
    del wl
    torch.cuda.empty_cache()
    peak, measured = int8_peak_tops()
    wl = PrefillSweep(torch, ctx)
    ms = timed_steps(torch, wl, 2, warmup=1)
    cases = wl.per_case(min_ms=10.0)
    agg = wl.ops_per_step / (ms * 1e-3) / 1e12
    worst = min(cases, key=lambda c: c["tops"])
    best = max(cases, key=lambda c: c["tops"])
    out["configs2_prefill"] = {
        "aggregate_tops": round(agg, 1), "aggregate_frac_of_int8_peak": round(agg / peak, 3),
        "best": dict(best, frac=round(best["tops"] / peak, 3)), "worst": dict(worst, frac=round(worst["tops"] / peak, 3)),
        "int8_peak_tops": round(peak, 1), "int8_peak_source": "2 x measured bf16 burst" if measured else "2 x fallback bf16",
        "library_int8_tops_8192cubed": int8_library_tops(torch),
        "cases": [[c["name"], c["M"], c["g"], c["us"], c["tops"]] for c in cases]}
    wl.close()
    del wl
    torch.cuda.empty_cache()
    wl = FastARFrame(torch, ctx)
    ms = timed_steps(torch, wl, 20)
    gbs = wl.bytes_per_step / (ms * 1e-3) / 1e9
    out["configs4_fast_ar_frame"] = {"ms_per_frame": round(ms, 4), "codebook_tokens_per_s": round(wl.batch * wl.codebooks / (ms * 1e-3), 1),
                                     "frame_gbs": round(gbs, 1), "frac_of_hbm": round(gbs / hbm, 3),
                                     "lm_head_int8_155776": wl.lm_head()}
    wl.close()
    del wl
    torch.cuda.empty_cache()
    return out


def agreed_top_up_steps(torch, dist, remaining_s, step_s, device):
    """How many more steps every rank runs so that about `remaining_s` more seconds of load are seen: each rank brings
    its own clock reading and step time, all leave with the same count (the largest remaining time over the largest
    step time, at least one step if any rank has time left). dist None: a single process."""
    plan = torch.tensor([max(0.0, remaining_s), step_s], dtype=torch.float64, device=device)
    if dist is not None:
        dist.all_reduce(plan, op=dist.ReduceOp.MAX)
    remaining, step = plan.tolist()
    return int(remaining / max(step, 1e-5)) + 1 if remaining > 0 else 0


def finish(dist, wl):
    """Leaves a multi-rank job without tearing NCCL down: a communicator destroyed while captured graphs
    that used it are alive has hung at exit, so graphs go first and the process exits hard."""
    import torch

    torch.cuda.synchronize()
    if dist is None:
        return
    getattr(wl, "graphs", {}).clear()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


REFERENCE_SAMPLE = ("the reference's own CUDA kernels (rebuilt for sm_100, stock entry points) on the GPU, eager "
                    "launches: the reference has no CPU implementation of this path")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=["decode_stack", "decode_sweep", "prefill", "fast_ar", "config0"],
                    default="decode_stack")
    ap.add_argument("--tp-mode", choices=["fused", "nccl"], default="fused",
                    help="N > 1: all-reduce inside the norm kernel over peer memory (fused) or NCCL (baseline)")
    ap.add_argument("--layers", type=int, default=36, help="decode_stack: number of layers (36 = the named config)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only", default=None, metavar="NAME:M:G",
                    help="restrict the sweep to one case, e.g. gate_up:16:256 (for profiling)")
    ap.add_argument("--no-detail", action="store_true", help="skip the per-case timings and the extra configurations")
    ap.add_argument("--split-k", type=int, default=0, help="force the GEMV's K-slice count (tuning aid)")
    ap.add_argument("--no-pack", action="store_true", help="leave weights row-major (skip the loader-side pack)")
    ap.add_argument("--eager", action="store_true", help="launch kernels one by one instead of replaying a graph")
    ap.add_argument("--trace", action="store_true",
                    help="decode_stack: add the per-kernel device timeline of one replayed step to the line; prefill: add "
                         "the per-K-group timeline of the GEMM's MMA lane, epilogue and producer (both need a library "
                         "built with --define W8A8_TRACE, named by W8A8_LIBRARY)")
    ap.add_argument("--timeline", action="store_true",
                    help="with --step-form one-launch: add the device-side per-phase medians of one step to the line")
    ap.add_argument("--step-form", choices=["one-launch", "chain"], default="chain",
                    help="decode_stack on one GPU: the whole step as one persistent kernel (w8a8_decode_stack_step) "
                         "or as a chain of launches per layer")
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
    if world > 1 and args.impl == "reference":
        # the reference has no multi-GPU path: rank 0 alone runs it, the others leave at once
        if rank != 0:
            return
        world = 1
        declared_world = int(os.environ.get("WORLD_SIZE", "1"))
    else:
        declared_world = world
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    pkg = ge.package()
    reference = args.impl == "reference"
    ctx = None
    if reference:
        from oracle import fishref

        if not fishref.available():
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable":
                                  "oracle/_ref/libfishref.so was not built (no reference checkout at build time)"}))
            return
        # nothing of the product is loaded on this arm: weights, cache and inputs are made with torch alone
        if args.workload == "decode_stack":
            wl = DecodeStack(torch, None, 1, 0, None, layers=args.layers, reference=True)
        elif args.workload == "prefill":
            wl = PrefillSweep(torch, None, reference=True)
        elif args.workload == "fast_ar":
            wl = FastARFrame(torch, None, reference=True)
        elif args.workload == "config0":
            wl = DecodeSweep(torch, None, reference=True, cases=config0_cases())
        else:
            wl = DecodeSweep(torch, None, reference=True)
    else:
        ctx = pkg.Context(local_rank, 0)
        if args.workload == "decode_stack":
            wl = DecodeStack(torch, ctx, world, rank, dist, layers=args.layers, tp_mode=args.tp_mode)
        elif args.workload == "prefill":
            wl = PrefillSweep(torch, ctx)
        elif args.workload == "fast_ar":
            wl = FastARFrame(torch, ctx)
        elif args.workload == "config0":
            wl = DecodeSweep(torch, ctx, pack=not args.no_pack, cases=config0_cases())
        else:
            wl = DecodeSweep(torch, ctx, pack=not args.no_pack)

    wl.eager = args.eager
    if args.workload == "decode_stack" and not reference and world == 1:
        wl.one_launch = args.step_form == "one-launch"
        if wl.one_launch:
            wl.launches_per_step = 1
    wl.split_k = args.split_k

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # The clock record covers everything that runs under load from the first warm-up step on: warm-up, the timed
    # region, the end-to-end region, the dominant kernel timed alone; a short run keeps stepping until the sampler
    # has seen about 1.5 s of load.
    # All ranks leave set-up together: the first (eager) step of a tensor-parallel stack waits in every exchange for
    # the peers' rows, and a rank that enters it seconds before a peer has finished packing its weights sits out one
    # bounded wait per exchange (72 per step, seconds each) before the run gets going.
    barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    t_load0 = time.perf_counter()
    for _ in range(args.warmup):
        wl.step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(args.steps):
        wl.step()
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    # end to end: host buffers in, host buffers out, copies inside the timed region
    e2e_ms = None
    if not reference and args.workload != "prefill":
        for _ in range(2):
            wl.step(e2e=True)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            wl.step(e2e=True)
        barrier()
        e2e_ms = (time.perf_counter() - t0) * 1e3
    cases = [] if args.no_detail else wl.per_case()
    lin = wl.time_linears() if (args.workload == "decode_stack" and not reference) else None
    # Keep stepping until the sampler has seen about 1.5 s of load. Every rank must run the SAME number of steps: a
    # tensor-parallel step that one rank runs alone waits out every one of its exchanges (72 bounded waits of seconds
    # each) and leaves that rank's exchange epoch ahead of its peers' for good. So the count is agreed first.
    for _ in range(agreed_top_up_steps(torch, dist, 1.5 - (time.perf_counter() - t_load0),
                                       dev_ms / max(args.steps, 1) * 1e-3, "cuda")):
        wl.step()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    # every rank steps (the tensor-parallel exchange needs all of them); rank 0 reports its own GPU's timeline
    kernel_timeline = None
    if args.trace and args.workload == "decode_stack" and not reference:
        barrier()
        kernel_timeline = step_timeline(torch, wl)
        barrier()

    times = torch.tensor([dev_ms, e2e_ms or 0.0, lin[0] if lin else 0.0], dtype=torch.float64, device="cuda")
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms_max, lin_s = times.tolist()
    if rank != 0:
        finish(dist, wl)
        return

    pk = peaks()
    ms_per_step = dev_ms / args.steps
    par = f"replicas x{world}" if world > 1 else "single GPU"
    if reference:
        par = "single GPU (the reference has no multi-GPU path; rank 0 alone ran)"

    def reference_keys(line, unit):
        line["impl"] = "reference"
        line["n_gpus"] = declared_world
        line["gpu_launches"] = None
        line["cpu_baseline"] = {"value": line["value"], "unit": unit, "cores": 0, "kind": "reference",
                                "sample": REFERENCE_SAMPLE}
        line["e2e"] = {"value": line["value"], "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}

    if args.workload == "prefill":
        tops = wl.ops_per_step * world / (ms_per_step * 1e-3) / 1e12
        peak, measured = int8_peak_tops()
        line = {
            "metric": "w8a8_prefill_gemm_int8_tops", "value": round(tops, 1), "unit": "TOPS", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "configs[2]: slow-AR projections qkv/o/gate_up/down x g{256,64} x M{2048,8192}, one "
                                   "W8A8 linear (row quantiser + tcgen05 GEMM) each per step", "cases_per_step": len(wl.cases),
                       "l2": "inputs larger than L2: 8 weight sets + 8 activation sets in rotation (> 600 MB)",
                       "parallelism": par,
                       "library_int8_tops_8192cubed": int8_library_tops(torch),
                       **({"gemm_timeline": gemm_timeline(torch, ge.package())} if (args.trace and not reference) else {})},
            "roofline": {"bound": "tensor", "achieved": round(tops / world, 1), "peak": round(peak, 1), "unit": "TOP/s",
                         "frac": round(tops / world / peak, 4),
                         "traffic": int(GEMM_TRAFFIC_RATIO * sum(
                             c["N"] * c["K"] + 2 * c["N"] * (c["K"] // c["g"]) + c["M"] * c["K"]
                             + 4 * c["M"] * (c["K"] // c["g"]) + 2 * c["M"] * c["N"] for c in wl.cases) / len(wl.cases)),
                         "traffic_source": "bytes per launch (mean over the cases) scaled by the DRAM/algorithmic ratio "
                                           "of one ncu capture (gate_up M=2048 g=256)",
                         "peak_source": "2 x measured bf16 burst (int8 dense runs at twice the bf16 rate; no "
                                        "int8 figure is in MEASURED_PEAKS.json)" if measured else "2 x fallback bf16",
                         "kernel": "gemm_i8_kernel" if not reference else "reference kernels (per-group cuBLAS + accumulate)"},
            "clocks": clocks, "gpu_launches": wl.launches_per_step * args.steps,
            "cases": [dict(c, frac=round(c["tops"] / peak, 3)) for c in cases],
            "e2e": {"value": None, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "prefill activations are produced on the device by the embedding / previous layer; "
                            "the end-to-end figure of this repository is the decode_stack workload's"},
        }
        if reference:
            line["roofline"]["traffic"] = None
            reference_keys(line, "TOPS")
        elif not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_prefill()
        print(json.dumps(line), flush=True)
        finish(dist, wl)
        return
    if args.workload == "fast_ar":
        tok_s = wl.batch * wl.codebooks / (ms_per_step * 1e-3)
        gbs = wl.bytes_per_step / (ms_per_step * 1e-3) / 1e9
        line = {
            "metric": "fast_ar_codebook_tokens_per_s", "value": round(tok_s * world, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": "configs[4]: fast-AR codebook decoder, one frame per step = 10 codebook steps x (4 layers, "
                                   "hidden 2560, 32q/8kv x128, SwiGLU 9728, no qk-norm, W8A8 g64) + codebook head 2560->4096, "
                                   "batch 8; sampling and embedding lookup outside; one CUDA graph per frame",
                       "global_batch": wl.batch, "codebooks": wl.codebooks,
                       "parallelism": par,
                       "l2": "a frame streams 10 x 0.42 GB of weights: each codebook step's weights exceed L2",
                       "lm_head_int8_155776": None if (args.no_detail or reference) else wl.lm_head()},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(gbs / pk["hbm_gbs"], 4), "traffic": None, "peak_source": pk["source"],
                         "kernel": "the whole frame (weights + scales + KV read, algorithmic bytes over frame time)"},
            "clocks": clocks, "gpu_launches": wl.launches_per_step * args.steps,
        }
        if reference:
            reference_keys(line, "tokens/s")
        else:
            line["roofline"]["algorithmic_bytes_per_launch"] = int(wl.bytes_per_step / wl.launches_per_step)
            line["e2e"] = {"value": round(wl.batch * wl.codebooks / (e2e_ms_max / args.steps * 1e-3), 1), "unit": "tokens/s",
                           "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h}
        print(json.dumps(line), flush=True)
        finish(dist, wl)
        return
    if args.workload == "decode_stack":
        n_gpus = world
        tok_s = wl.batch / (ms_per_step * 1e-3)
        line = {
            "metric": "slow_ar_decode_tokens_per_s", "value": round(tok_s, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
            "config": {"workload": f"configs[3]: slow-AR decoder stack, {args.layers} layers, hidden 2560, 32q/8kv x128, "
                                   "SwiGLU 9728, W8A8 g256, fp16 paged KV (16-token blocks), batch 8, context 1024, "
                                   "random-init weights; LM head and sampling outside the step",
                       "global_batch": wl.batch, "context": wl.context,
                       "parallelism": f"tp{n_gpus}" + ((" (all-reduce after wo and w2 fused into the norm kernel over NVLink peer "
                                                              "memory)" if wl.tp_mode == "fused" else
                                                              " (NCCL fp16 all-reduce after wo and w2)") if n_gpus > 1 else ""),
                       "l2": "inputs larger than L2: a step streams 3.6 GB of weights + 1.2 GB of KV",
                       "step_hbm_gbs_per_gpu": round(wl.bytes_per_step / (ms_per_step * 1e-3) / 1e9, 1),
                       "step_hbm_frac_per_gpu": round(wl.bytes_per_step / (ms_per_step * 1e-3) / 1e9 / pk["hbm_gbs"], 4)},
            "clocks": clocks,
            "gpu_launches": wl.launches_per_step * args.steps,
        }
        if args.timeline and getattr(wl, "one_launch", False):
            line["config"]["timeline_us"] = wl.timeline()
        if kernel_timeline is not None:
            line["config"]["kernel_timeline"] = kernel_timeline
        if lin:
            ach = lin[1] / lin_s / 1e9
            line["roofline"] = {"bound": "hbm", "achieved": round(ach, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                                "frac": round(ach / pk["hbm_gbs"], 4),
                                "traffic": int(GEMV_TRAFFIC_RATIO * lin[1]),
                                "traffic_source": "algorithmic bytes per launch scaled by the DRAM/algorithmic ratio of "
                                                  "one ncu capture (w1|w3 at M=8 g=256)",
                                "peak_source": pk["source"],
                                "kernel": "gemv_packed_kernel (the 4 linears of each layer, timed alone)",
                                "algorithmic_bytes_per_launch": int(lin[1]), "us_per_launch": round(lin_s * 1e6, 2)}
        if reference:
            reference_keys(line, "tokens/s")
            line["config"]["parallelism"] = par
        else:
            line["e2e"] = {"value": round(wl.batch / (e2e_ms_max / args.steps * 1e-3), 1), "unit": "tokens/s",
                           "h2d_bytes_per_step": wl.h2d, "d2h_bytes_per_step": wl.d2h}
            if not args.no_cpu_baseline:
                line["cpu_baseline"] = cpu_baseline_stack()
            if world == 1 and not args.no_detail and args.layers == 36:
                wl.close()
                del wl
                torch.cuda.empty_cache()
                wl = None
                line["extra"] = extra_metrics(torch, ctx, pk)
        print(json.dumps(line), flush=True)
        finish(dist, wl)
        return
    # decode_sweep / config0
    total_bytes = wl.bytes_per_step * world
    value = total_bytes / (ms_per_step * 1e-3) / 1e9
    per_launch_bytes = wl.bytes_per_step / len(wl.cases)
    per_launch_s = ms_per_step * 1e-3 / len(wl.cases)
    achieved = per_launch_bytes / per_launch_s / 1e9
    what = ("configs[0]: one W8A8 linear, the gate projection, M=16 K=2560 N=9728 g=256" if args.workload == "config0" else
            "configs[1]: slow-AR projections qkv/o/gate_up/down x g{256,64} x M{1,4,16}, one W8A8 linear each per step")
    line = {
        "metric": "w8a8_decode_gemv_hbm_gbs", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_per_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": what, "cases_per_step": len(wl.cases),
                   "l2": "inputs larger than L2: >= 320 MB of copies per weight set in rotation, M outermost",
                   "parallelism": par,
                   "tops": round(wl.ops_per_step * world / (ms_per_step * 1e-3) / 1e12, 2)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4),
                     "traffic": None if reference else int(GEMV_TRAFFIC_RATIO * per_launch_bytes),
                     "peak_source": pk["source"],
                     "kernel": "gemv_packed_kernel" if not reference else "reference kernels",
                     "algorithmic_bytes_per_launch": int(per_launch_bytes)},
        "clocks": clocks,
        "gpu_launches": wl.launches_per_step * args.steps,
        "cases": [dict(c, frac=round(c["gbs"] / pk["hbm_gbs"], 3)) for c in cases],
    }
    if reference:
        reference_keys(line, "GB/s")
    else:
        e2e_value = total_bytes / (e2e_ms_max / args.steps * 1e-3) / 1e9
        line["e2e"] = {"value": round(e2e_value, 1), "unit": "GB/s", "h2d_bytes_per_step": wl.h2d,
                       "d2h_bytes_per_step": wl.d2h}
        if not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_sweep()
    print(json.dumps(line), flush=True)
    finish(dist, wl)


if __name__ == "__main__":
    main()
