#!/usr/bin/env python3
"""Benchmark of the IQ3_S x q8 MoE feed-forward path on B200.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N = 1 workload ("config 1" of the benchmark definition): one MoE layer, decode
batch 1 -- RMSNorm -> fp32 router (512 x 2048) -> softmax/top-10 -> 10 routed
IQ3_S experts + 1 shared expert (hidden 2048, intermediate 512).  One step is one
token through one layer.  Consecutive steps use different layers (48 distinct
layers of seeded synthetic weights, 33 GB resident in HBM) so no step finds its
weights in L2.  Metric: layer-tokens per second.

Printed: one JSON line (see the keys below).  `value` is timed with inputs
resident on the device; `e2e` goes through the same C-ABI call with the token's
hidden state copied from pinned host memory and the result read back every
step.  `cpu_baseline` times the reference engine's own CPU path for the same
layer on this host's cores.  `--impl reference` prints that CPU arm alone.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import __graft_entry__ as entry  # noqa: E402

N_EMBD, N_FF, N_EXPERT, TOPK = 2048, 512, 512, 10
EPS = 1e-6
IQ3S_BLOCK = 110
PACK = 2 * N_FF * (N_EMBD // 256) * IQ3S_BLOCK + N_EMBD * (N_FF // 256) * IQ3S_BLOCK  # 1351680
ROUTER_BYTES = N_EXPERT * N_EMBD * 4
# algorithmic bytes of one layer-token: router + (top-k + shared) expert packs
STEP_BYTES = ROUTER_BYTES + (TOPK + 1) * PACK
METRIC = "moe_layer_decode_tokens_per_s"
UNIT = "layer-tok/s"


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for i, nm in enumerate(names):
                    if r[5 + i].lower().startswith("active"):
                        reasons.add(nm)
            except Exception:
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


class Workload:
    """48 layers of synthetic weights generated on the device."""

    def __init__(self, pkg, n_layers, seed=2026):
        self.pkg = pkg
        self.dev = pkg.Device()
        lib = self.lib = self.dev.lib
        self.n_layers = n_layers
        self.slots_per_layer = N_EXPERT + 1
        n_slots = n_layers * self.slots_per_layer
        if not lib.q4_hip_experts_alloc_a(0, n_slots, PACK):
            raise MemoryError("expert arena of %d slots" % n_slots)
        self.base = lib.q4_hip_experts_base_a(0)
        self.stride = lib.q4_hip_experts_stride_a(0)
        assert lib.q4_cuda_synth_iq3s(self.base, n_slots * (PACK // IQ3S_BLOCK), seed)
        self.tiled = bool(lib.q4_cuda_experts_tiled_a(0))
        if self.tiled:      # generated in the engine's byte order: convert to the resident format
            assert lib.q4_cuda_experts_retile_a(0, 0, n_slots)
        self.d_router = self.dev.malloc(n_layers * ROUTER_BYTES)
        assert lib.q4_cuda_synth_normal(self.d_router, n_layers * N_EXPERT * N_EMBD, seed + 1, 0.0, 0.02)
        self.d_norm = self.dev.malloc(n_layers * N_EMBD * 4)
        assert lib.q4_cuda_synth_normal(self.d_norm, n_layers * N_EMBD, seed + 2, 1.0, 0.1)
        self.n_x = 64
        self.x_host = pkg.synth.hidden(seed + 3, self.n_x, N_EMBD)
        self.d_xpool = self.dev.upload(self.x_host)
        self.d_x = self.dev.malloc(N_EMBD * 4)
        self.d_y = self.dev.malloc(N_EMBD * 4)
        self.d_ids = self.dev.malloc(64 * 4)
        self.d_wts = self.dev.malloc(64 * 4)
        rb = N_EMBD // 256 * IQ3S_BLOCK
        self.og, self.ou, self.od = 0, N_FF * rb, 2 * N_FF * rb
        # pinned staging for the end-to-end leg
        self.h_x = lib.q4_hip_host_alloc_coh(N_EMBD * 4)
        self.h_y = lib.q4_hip_host_alloc_coh(N_EMBD * 4)
        self.dev.sync()

    def layer_base(self, l):
        return self.base + l * self.slots_per_layer * self.stride

    def step(self, i, d_x):
        l = i % self.n_layers
        ok = self.lib.q4_cuda_moe_decode(
            self.layer_base(l), self.stride, self.og, self.ou, self.od, N_EXPERT, d_x,
            self.d_norm + l * N_EMBD * 4, EPS, self.d_router + l * ROUTER_BYTES, N_EXPERT, TOPK,
            N_EMBD, N_FF, self.d_y, self.d_ids, self.d_wts)
        if not ok:
            raise RuntimeError("q4_cuda_moe_decode refused")

    def capture(self, g_steps):
        """CUDA graphs of g_steps consecutive steps each (one layer per step), enough
        of them to visit every layer, so that the device-resident leg is not paced
        by the host's launch loop."""
        self.g_steps = g_steps
        self.graphs = []
        n_var = (self.n_layers + g_steps - 1) // g_steps
        for v in range(n_var):
            assert self.lib.q4_hip_graph_begin() == 1
            for i in range(v * g_steps, (v + 1) * g_steps):
                self.step(i, self.d_xpool + (i % self.n_x) * N_EMBD * 4)
            g = self.lib.q4_hip_graph_end()
            if not g:
                raise RuntimeError("graph capture failed")
            self.graphs.append(g)

    def run_resident(self, n_graphs, first=0):
        for r in range(first, first + n_graphs):
            if not self.lib.q4_hip_graph_launch(self.graphs[r % len(self.graphs)]):
                raise RuntimeError("graph launch failed")

    def run_e2e(self, steps, first=0):
        import ctypes
        lib = self.lib
        for i in range(first, first + steps):
            l = i % self.n_layers
            ctypes.memmove(self.h_x, self.x_host[i % self.n_x].ctypes.data, N_EMBD * 4)
            ok = lib.q4_cuda_moe_decode_host(
                self.layer_base(l), self.stride, self.og, self.ou, self.od, N_EXPERT, self.h_x,
                self.d_norm + l * N_EMBD * 4, EPS, self.d_router + l * ROUTER_BYTES, N_EXPERT,
                TOPK, N_EMBD, N_FF, self.h_y)
            if not ok:
                raise RuntimeError("q4_cuda_moe_decode_host refused")

    def host_layers(self, n):
        """Copies of the first n layers' tensors on the host (for the CPU arm)."""
        out = []
        for l in range(n):
            packs = np.empty((self.slots_per_layer, PACK), np.uint8)
            for e in range(self.slots_per_layer):   # engine byte order, whatever the arena holds
                assert self.lib.q4_cuda_experts_get_a(0, l * self.slots_per_layer + e,
                                                      packs[e].ctypes.data, PACK)
            out.append({
                "experts": packs[:N_EXPERT], "shared": packs[N_EXPERT],
                "router": self.dev.download(self.d_router + l * ROUTER_BYTES, (N_EXPERT, N_EMBD), np.float32),
                "norm_w": self.dev.download(self.d_norm + l * N_EMBD * 4, (N_EMBD,), np.float32)})
        return out


def host_synth_layers(pkg, n, seed=2026):
    return [pkg.synth.layer(seed + 17 * l, N_EXPERT, N_EMBD, N_FF) for l in range(n)]


def cpu_arm(pkg, layers, x_host, budget_s):
    """Time the reference's CPU path (oracle/_ref) for whole layer-tokens."""
    from oracle import pyoracle
    ref = pyoracle.reference()
    kind = "reference"
    if ref is None:
        return None
    ncpu = os.cpu_count() or 2
    os.environ.setdefault("Q4_CPU_THREADS", str(max(1, min(16, ncpu - 1))))
    os.environ.setdefault("OMP_NUM_THREADS", str(max(1, min(16, ncpu - 1))))
    t, _, _ = ref.time_layers(layers, TOPK, 4, x_host, N_EMBD, N_FF, EPS)  # warm-up, pool start
    per = max(t / 4, 1e-5)
    jobs = int(max(16, min(20000, budget_s / per)))
    t, _, _ = ref.time_layers(layers, TOPK, jobs, x_host, N_EMBD, N_FF, EPS)
    return {"value": jobs / t, "unit": UNIT, "cores": ref.threads(), "kind": kind,
            "sample": "%d layer-tokens over %d layers (%.1f s), router+top-k on the host, "
                      "experts on the reference's worker pool" % (jobs, len(layers), t),
            "ms_per_step": 1e3 * t / jobs, "jobs": jobs}


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=200)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=48)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true")
    a = ap.parse_args()
    rank, world, local = dist_setup(a.gpus)
    warmup = max(a.warmup, 3)

    entry.build()
    pkg = entry.load_package()
    config = {"workload": "config1: one MoE layer, decode batch 1, hidden 2048, ff 512, "
                          "512 experts top-10 + shared, IQ3_S x q8",
              "layers_rotated": a.layers, "l2": "inputs larger than L2: every step reads a "
              "different layer (router+shared weights of all layers exceed L2)",
              "algorithmic_bytes_per_step": STEP_BYTES}

    if a.impl == "reference":
        if rank != 0:
            return
        layers = host_synth_layers(pkg, 2)
        x = pkg.synth.hidden(7, 64, N_EMBD)
        # K steps, each a bounded sample of the workload
        from oracle import pyoracle
        ref = pyoracle.reference()
        if ref is None:
            print(json.dumps({"impl": "reference", "unavailable":
                              "compiled reference CPU path (oracle/_ref) not present"}))
            return
        ncpu = os.cpu_count() or 2
        os.environ.setdefault("Q4_CPU_THREADS", str(max(1, min(16, ncpu - 1))))
        os.environ.setdefault("OMP_NUM_THREADS", str(max(1, min(16, ncpu - 1))))
        per_step = 64
        ref.time_layers(layers, TOPK, 8, x, N_EMBD, N_FF, EPS)
        steps = min(a.steps, 200)
        for _ in range(min(warmup, 3)):
            ref.time_layers(layers, TOPK, per_step, x, N_EMBD, N_FF, EPS)
        t = 0.0
        for _ in range(steps):
            dt, _, _ = ref.time_layers(layers, TOPK, per_step, x, N_EMBD, N_FF, EPS)
            t += dt
        val = steps * per_step / t
        line = {"impl": "reference", "metric": METRIC, "value": val, "unit": UNIT,
                "n_gpus": a.gpus, "steps": steps, "warmup": warmup,
                "ms_per_step": 1e3 * t / steps, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "int8 x IQ3_S, fp32 accumulate", "data": "synthetic",
                "config": dict(config, sample="%d layer-tokens per step over 2 layers" % per_step),
                "cpu_baseline": {"value": val, "unit": UNIT, "cores": ref.threads(),
                                 "kind": "reference",
                                 "sample": "%d steps x %d layer-tokens" % (steps, per_step)},
                "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if world > 1:
        raise SystemExit("multi-GPU expert-parallel arm is not built yet")

    wl = Workload(pkg, a.layers)
    lib = wl.lib
    launches0 = lib.q4_cuda_launch_count()
    # graph length: the largest divisor of the step count that is <= the layer count,
    # so that exactly `steps` steps are timed
    g_steps = max(d for d in range(1, a.layers + 1) if a.steps % d == 0)
    wl.capture(g_steps)
    launches_per_step = (lib.q4_cuda_launch_count() - launches0) / (len(wl.graphs) * g_steps)
    n_graphs = a.steps // g_steps
    wl.run_resident((warmup + g_steps - 1) // g_steps)
    wl.dev.sync()

    sampler = ClockSampler(local)
    sampler.start()
    # --- device-resident throughput ---
    wl.dev.sync()
    lib.q4_cuda_timer_begin()
    wl.run_resident(n_graphs)
    lib.q4_cuda_timer_end()
    ms = lib.q4_cuda_timer_ms()
    wl.dev.sync()
    # --- end to end through the C ABI with host buffers ---
    wl.run_e2e(min(warmup, 50))
    lib.q4_cuda_timer_begin()
    t0 = time.perf_counter()
    wl.run_e2e(a.steps, first=warmup)
    lib.q4_cuda_timer_end()
    ms_e2e_dev = lib.q4_cuda_timer_ms()
    ms_e2e = max(ms_e2e_dev, 1e3 * (time.perf_counter() - t0))
    clocks = sampler.stop()
    err = lib.q4_cuda_device_error()
    if err:
        raise SystemExit("device error word %#x" % err)

    peak, peak_src = read_peaks()
    per_launch_s = ms * 1e-3 / a.steps
    achieved = STEP_BYTES / per_launch_s / 1e9
    cpu = None
    if not a.no_cpu:
        cpu = cpu_arm(pkg, wl.host_layers(2), wl.x_host, a.cpu_seconds)
    line = {
        "metric": METRIC, "value": a.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": a.steps, "warmup": warmup, "ms_per_step": ms / a.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x IQ3_S, fp32 accumulate", "data": "synthetic", "config": config,
        "clocks": clocks,
        "e2e": {"value": a.steps / (ms_e2e * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": N_EMBD * 4, "d2h_bytes_per_step": N_EMBD * 4},
        "gpu_launches": int(round(launches_per_step * a.steps * 2)),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_source": peak_src,
                     "kernel": "whole step (%g launches/step)" % launches_per_step},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
