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

# CPU arm: the reference's expert pool gets the cores; its small host-side router GEMV (OpenMP in
# the reference's build) stays on one thread -- an OpenMP team next to the pool's spinning workers
# was measured 13x slower.  Must be set before the OpenMP runtime is loaded.
os.environ["OMP_NUM_THREADS"] = os.environ.get("Q4B_REF_OMP", "1")

import numpy as np  # noqa: E402

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
# DRAM bytes of one launch of the persistent decode kernel, from an ncu capture of this
# workload (read 19,163,136 + write 0..256); the algorithmic figure is STEP_BYTES
FUSED_DRAM_BYTES_PER_LAUNCH = 19159040
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
        self.y_out = np.zeros(N_EMBD, np.float32)
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

    def capture_tail(self, n):
        """One more graph of n < g_steps steps: the remainder when the step count is not a
        multiple of the graph length."""
        self.tail = None
        if n:
            assert self.lib.q4_hip_graph_begin() == 1
            for i in range(n):
                self.step(i, self.d_xpool + (i % self.n_x) * N_EMBD * 4)
            self.tail = self.lib.q4_hip_graph_end()
            if not self.tail:
                raise RuntimeError("graph capture failed")

    def run_resident(self, n_graphs, first=0, tail=False):
        for r in range(first, first + n_graphs):
            if not self.lib.q4_hip_graph_launch(self.graphs[r % len(self.graphs)]):
                raise RuntimeError("graph launch failed")
        if tail and self.tail and not self.lib.q4_hip_graph_launch(self.tail):
            raise RuntimeError("graph launch failed")

    def run_e2e(self, steps, first=0):
        """Per step: the token's row is written into pinned host memory, the layer runs through the
        host-buffer call (arguments bound once per layer), the 8 KB result is read on the host."""
        import ctypes
        lib = self.lib
        if not hasattr(self, "plans"):
            self.plans = []
            for l in range(self.n_layers):
                p = lib.q4_cuda_decode_plan(self.layer_base(l), self.stride, self.og, self.ou, self.od,
                                            N_EXPERT, self.d_norm + l * N_EMBD * 4, EPS,
                                            self.d_router + l * ROUTER_BYTES, N_EXPERT, TOPK, N_EMBD, N_FF)
                if not p:
                    raise RuntimeError("q4_cuda_decode_plan refused")
                self.plans.append(p)
        run, h_x, h_y = lib.q4_cuda_decode_plan_host, self.h_x, self.h_y
        for i in range(first, first + steps):
            ctypes.memmove(h_x, self.x_host[i % self.n_x].ctypes.data, N_EMBD * 4)
            ok = run(self.plans[i % self.n_layers], h_x, h_y)
            if not ok:
                raise RuntimeError("q4_cuda_decode_plan_host refused")
            ctypes.memmove(self.y_out.ctypes.data, self.h_y, N_EMBD * 4)   # the step's result, read on the host

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


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


def cpu_arm(pkg, layers, x_host, budget_s):
    """Time the reference's CPU path (oracle/_ref) for whole layer-tokens."""
    from oracle import pyoracle
    ref = pyoracle.reference()
    kind = "reference"
    if ref is None:
        return None
    ncpu = os.cpu_count() or 2
    os.environ.setdefault("Q4_CPU_THREADS", str(max(1, min(16, ncpu - 1))))
    t, _, _ = ref.time_layers(layers, TOPK, 4, x_host, N_EMBD, N_FF, EPS)  # warm-up, pool start
    per = max(t / 4, 1e-5)
    jobs = int(max(16, min(20000, budget_s / per)))
    t, _, _ = ref.time_layers(layers, TOPK, jobs, x_host, N_EMBD, N_FF, EPS)
    return {"value": jobs / t, "unit": UNIT, "cores": ref.threads(), "kind": kind, "cpu_model": cpu_model(),
            "sample": "%d layer-tokens over %d layers (%.1f s), router+top-k on the host, "
                      "experts on the reference's worker pool" % (jobs, len(layers), t),
            "ms_per_step": 1e3 * t / jobs, "jobs": jobs}


def exchange_id(rank, world, make_id):
    """Rank 0 makes the 128-byte communicator id; the others fetch it over a local socket."""
    import socket
    port = (int(os.environ.get("MASTER_PORT", "29500")) + 1000) % 65536 or 30500
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    if rank == 0:
        ident = make_id()
        srv = socket.socket()
        srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        srv.bind((addr, port))
        srv.listen(world)
        for _ in range(world - 1):
            c, _ = srv.accept()
            c.sendall(ident)
            c.close()
        srv.close()
        return ident
    deadline = time.time() + 120
    while True:
        try:
            c = socket.create_connection((addr, port), timeout=5)
            break
        except OSError:
            if time.time() > deadline:
                raise
            time.sleep(0.2)
    buf = b""
    while len(buf) < 128:
        chunk = c.recv(128 - len(buf))
        if not chunk:
            raise RuntimeError("id exchange broke")
        buf += chunk
    c.close()
    return buf


EP_TOKENS = 64          # config 4: batch of 64 tokens ...
EP_LAYERS = 48          # ... through 48 MoE layers


class EpJob:
    """64 tokens x n_layers MoE layers on `world` ranks; this object is one rank's part.
    world == 1 is the same job on one GPU through q4_cuda_moe_layer_n."""

    def __init__(self, pkg, dev, ep, arena, rank, world, n_layers, tokens=EP_TOKENS, zipf=False):
        import ctypes
        self.lib = lib = dev.lib
        if os.environ.get("Q4B_TC_MODE"):   # experiments: which grouped-product kernel runs (default: split by rows)
            assert lib.q4_cuda_mmq_tc_mode(int(os.environ["Q4B_TC_MODE"]))
        self.ep, self.world, self.n_layers, self.arena = ep, world, n_layers, arena
        self.tokens = tokens
        self.t_local = tokens // world
        e_local = self.e_local = N_EXPERT // world
        self.slots_l = e_local + 1
        bpp = PACK // IQ3S_BLOCK            # super-blocks per expert pack
        if not lib.q4_hip_experts_alloc_a(arena, n_layers * self.slots_l, PACK):
            raise MemoryError("expert arena")
        self.base, self.stride = lib.q4_hip_experts_base_a(arena), lib.q4_hip_experts_stride_a(arena)
        # expert (layer, e) has the same bytes at every world size: each rank generates
        # its range of the full seeded tensor, then the layer's shared expert
        for l in range(n_layers):
            lb = self.base + l * self.slots_l * self.stride
            first = (l * (N_EXPERT + 1) + rank * e_local) * bpp
            assert lib.q4_cuda_synth_iq3s_at(lb, e_local * bpp, 2026, first)
            assert lib.q4_cuda_synth_iq3s_at(lb + e_local * self.stride, bpp, 2026,
                                             (l * (N_EXPERT + 1) + N_EXPERT) * bpp)
        if lib.q4_cuda_experts_tiled_a(arena):
            assert lib.q4_cuda_experts_retile_a(arena, 0, n_layers * self.slots_l)
        self.d_router = dev.malloc(n_layers * ROUTER_BYTES)
        assert lib.q4_cuda_synth_normal(self.d_router, n_layers * N_EXPERT * N_EMBD, 2027, 0.0, 0.02)
        self.d_norm = dev.malloc(n_layers * N_EMBD * 4)
        assert lib.q4_cuda_synth_normal(self.d_norm, n_layers * N_EMBD, 2028, 1.0, 0.1)
        x_all = pkg.synth.hidden(2029, tokens, N_EMBD)
        if zipf:
            # Expert popularity skewed by a Zipf(1.1) bias on the router logits: every
            # token carries the same value A in coordinate 0 (norm weight 1 there), and
            # router column 0 holds bias_e / (normalised A), so logit_e = N(0, ~1) + bias_e.
            A = 4.0
            x_all[:, 0] = A
            xn0 = A / np.sqrt((A * A + N_EMBD - 1.0) / N_EMBD)
            col = (pkg.synth.zipf_bias(N_EXPERT, 1.1) / xn0).astype(np.float32)
            one = np.ones(1, np.float32)
            dev.sync()
            for l in range(n_layers):
                r = dev.download(self.d_router + l * ROUTER_BYTES, (N_EXPERT, N_EMBD), np.float32)
                r[:, 0] = col
                dev.write(self.d_router + l * ROUTER_BYTES, r)
                dev.write(self.d_norm + l * N_EMBD * 4, one)
        self.x_host = np.ascontiguousarray(x_all[rank * self.t_local:(rank + 1) * self.t_local])
        self.nb = nb = self.t_local * N_EMBD * 4
        self.d_x0, self.d_a, self.d_b = dev.upload(self.x_host), dev.malloc(nb), dev.malloc(nb)
        self.h_x, self.h_y = lib.q4_hip_host_alloc_coh(nb), lib.q4_hip_host_alloc_coh(nb)
        ctypes.memmove(self.h_x, self.x_host.ctypes.data, nb)
        rb = N_EMBD // 256 * IQ3S_BLOCK
        self.og, self.ou, self.od = 0, N_FF * rb, 2 * N_FF * rb
        if world == 1:
            self.ws = lib.q4_cuda_moe_layer_n_ws_bytes(self.t_local, TOPK, N_EXPERT, N_EMBD, N_FF)
        else:
            self.ws = ep.q4_cuda_ep_layer_ws_bytes(world, self.t_local, TOPK, N_EXPERT, N_EMBD, N_FF)
        self.d_ws = dev.malloc(self.ws)
        self.dev = dev
        self.graph = None

    def layer(self, l, src, dst):
        lb = self.base + l * self.slots_l * self.stride
        nw, rt = self.d_norm + l * N_EMBD * 4, self.d_router + l * ROUTER_BYTES
        if self.world == 1:
            ok = self.lib.q4_cuda_moe_layer_n(lb, self.stride, self.og, self.ou, self.od, N_EXPERT, src, nw,
                                              EPS, rt, N_EXPERT, TOPK, N_EMBD, N_FF, self.t_local, dst,
                                              None, None, self.d_ws, self.ws)
        else:
            ok = self.ep.q4_cuda_ep_layer(lb, self.stride, self.og, self.ou, self.od, 1, src, nw, EPS, rt,
                                          N_EXPERT, TOPK, N_EMBD, N_FF, self.t_local, dst, self.d_ws, self.ws)
        if not ok:
            raise RuntimeError("layer call refused")

    def enqueue(self):
        src = self.d_x0
        for l in range(self.n_layers):      # the output of a layer is the next layer's input
            dst = self.d_a if (l % 2 == 0) else self.d_b
            self.layer(l, src, dst)
            src = dst
        self.d_out = src

    def try_capture(self):
        """One CUDA graph per step (48 layers); falls back to plain launches if the capture
        is refused (e.g. by the collective library)."""
        if os.environ.get("Q4B_BENCH_GRAPH", "1") == "0":
            return False
        if self.lib.q4_hip_graph_begin() != 1:
            return False
        try:
            self.enqueue()
        except RuntimeError:
            self.lib.q4_hip_graph_end()
            return False
        g = self.lib.q4_hip_graph_end()
        if not g:
            return False
        self.graph = g
        return True

    def step(self):
        if self.graph:
            if not self.lib.q4_hip_graph_launch(self.graph):
                raise RuntimeError("graph launch failed")
        else:
            self.enqueue()

    def step_e2e(self):
        lib = self.lib
        lib.q4_hip_h2d_async(self.d_x0, self.h_x, self.nb)
        self.step()
        lib.q4_hip_d2h_async(self.h_y, self.d_out, self.nb)
        lib.q4_hip_stream_sync()

    def release(self):
        if self.graph:      # a graph that holds collective nodes must go before the communicator does
            self.lib.q4_hip_graph_free(self.graph)
            self.graph = None
        self.lib.q4_hip_experts_free_a(self.arena)
        for p in (self.d_router, self.d_norm, self.d_x0, self.d_a, self.d_b, self.d_ws):
            self.lib.q4_hip_free(p)


def time_job(job, steps, warmup, barrier_max):
    """(ms resident, ms end to end, launches per step) for `steps` steps, max over ranks."""
    lib = job.lib
    l0 = lib.q4_cuda_launch_count()
    job.enqueue()
    job.dev.sync()
    launches = lib.q4_cuda_launch_count() - l0
    job.try_capture()
    for _ in range(warmup):
        job.step()
    job.dev.sync()
    barrier_max(0.0)
    lib.q4_cuda_timer_begin()
    for _ in range(steps):
        job.step()
    lib.q4_cuda_timer_end()
    ms = barrier_max(lib.q4_cuda_timer_ms())
    job.dev.sync()
    for _ in range(2):
        job.step_e2e()
    barrier_max(0.0)
    lib.q4_cuda_timer_begin()
    t0 = time.perf_counter()
    for _ in range(steps):
        job.step_e2e()
    lib.q4_cuda_timer_end()
    ms_e2e = barrier_max(max(lib.q4_cuda_timer_ms(), 1e3 * (time.perf_counter() - t0)))
    return ms, ms_e2e, launches


def ep_roofline(world, n_layers, t_step):
    """HBM roofline of the expert-parallel job over all ranks: every rank reads the router of
    each layer and the packs of the distinct experts routed to it plus its copy of the shared
    expert.  The number of distinct routed experts per layer is the expectation for uniform
    routing, E * (1 - (1 - k/E)^T) = 367 of 512 at 64 tokens, not a count of this run."""
    hbm, src = read_peaks()
    distinct = N_EXPERT * (1.0 - (1.0 - TOPK / N_EXPERT) ** EP_TOKENS)
    per_layer = world * (ROUTER_BYTES + PACK) + distinct * PACK
    achieved = per_layer * n_layers / t_step / 1e9
    return {"bound": "hbm", "achieved": achieved, "peak": hbm * world, "unit": "GB/s",
            "frac": achieved / (hbm * world), "traffic": None, "peak_source": src + " x n_gpus",
            "kernel": "whole step, all ranks; expected distinct experts %.0f per layer" % distinct}


def run_ep(a, pkg, rank, world, local, warmup):
    """Config 4: expert-parallel decode, 64 tokens x 48 layers, experts sharded evenly,
    router and shared expert replicated, dispatch/combine over NCCL.  Strong scaling: the
    job (64 x 48 layer-tokens per step) is the same at every N.  Rank 0 afterwards runs the
    same job alone on its GPU so the line carries its own 1-GPU reference."""
    import ctypes
    dev = pkg.Device()
    lib = dev.lib
    ep = None
    if world > 1:
        ep = pkg.capi.load_ep()

        def make_id():
            buf = ctypes.create_string_buffer(128)
            assert ep.q4_cuda_ep_unique_id(buf)
            return buf.raw
        ident = exchange_id(rank, world, make_id)
        assert ep.q4_cuda_ep_init(ident, rank, world), "NCCL communicator"

    def barrier_max(v):
        if world == 1:
            return v
        f = ctypes.c_float(v)
        assert ep.q4_cuda_ep_allreduce_max(ctypes.byref(f))
        return f.value

    n_layers = a.layers if a.layers else EP_LAYERS
    job = EpJob(pkg, dev, ep, 0, rank, world, n_layers)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, ms_e2e, launches = time_job(job, a.steps, warmup, barrier_max)
    clocks = sampler.stop() if rank == 0 else None
    graphed = bool(job.graph)
    err = lib.q4_cuda_device_error()
    if err:
        raise SystemExit("device error word %#x" % err)
    single = None
    if world > 1 and rank == 0 and not a.no_cpu:
        job.release()
        solo = EpJob(pkg, dev, None, 0, 0, 1, n_layers)
        s_ms, s_e2e, _ = time_job(solo, a.steps, warmup, lambda v: v)
        single = {"value": EP_TOKENS * n_layers * a.steps / (s_ms * 1e-3),
                  "e2e": EP_TOKENS * n_layers * a.steps / (s_e2e * 1e-3), "unit": UNIT,
                  "ms_per_step": s_ms / a.steps}
    barrier_max(0.0)
    if rank == 0:
        units = EP_TOKENS * n_layers
        peak, peak_src = read_peaks()
        # weight bytes a step must read on the busiest rank: all routers + the experts picked
        print(json.dumps({
            "metric": METRIC, "value": units * a.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": a.steps, "warmup": warmup, "ms_per_step": ms / a.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 x IQ3_S, fp32 accumulate",
            "data": "synthetic",
            "config": {"workload": "config4: expert-parallel decode, 64 tokens x %d MoE layers per step, 512 "
                                   "experts top-10 + shared, experts sharded %d-way, NCCL dispatch/combine"
                                   % (n_layers, world),
                       "l2": "inputs larger than L2: a step reads %d layers of weights" % n_layers,
                       "tokens_per_rank": job.t_local, "experts_per_rank": job.e_local,
                       "cuda_graph": graphed, "one_gpu_same_job": single},
            "clocks": clocks,
            "e2e": {"value": units * a.steps / (ms_e2e * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": job.nb, "d2h_bytes_per_step": job.nb},
            "gpu_launches": int(launches * a.steps * 2),
            "roofline": ep_roofline(world, n_layers, ms * 1e-3 / a.steps), "cpu_baseline": None}))
    if ep:
        barrier_max(0.0)
        if job.graph:
            lib.q4_hip_graph_free(job.graph)
            job.graph = None
        # tearing the communicator down must not be able to hold the process: give it ten seconds
        t = threading.Thread(target=ep.q4_cuda_ep_shutdown, daemon=True)
        t.start()
        t.join(10.0)
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def run_batch(a, pkg, local, warmup, kind):
    """One GPU, many tokens per step through q4_cuda_moe_layer_n.
    verify  (config 2): 4 tokens (1 + 3 drafts) through 48 layers, y of a layer feeding the next.
    prefill (config 3): 2048 tokens through one layer, expert popularity skewed by Zipf(1.1);
                        consecutive steps alternate between two layers of weights."""
    dev = pkg.Device()
    lib = dev.lib
    if kind == "verify":
        tokens, n_layers, zipf = 4, (a.layers or 48), False
    else:
        tokens, n_layers, zipf = 2048, 2, True
    job = EpJob(pkg, dev, None, 0, 0, 1, n_layers, tokens=tokens, zipf=zipf)
    if kind == "prefill":
        # one layer per step: step i runs layer i % 2 on the same input rows
        job.enqueue_all = job.enqueue
        state = {"i": 0}

        def one_layer():
            job.layer(state["i"] % n_layers, job.d_x0, job.d_a)
            state["i"] += 1
            job.d_out = job.d_a
        job.enqueue = one_layer
        job.try_capture = lambda: False
    # routed rows and distinct experts of the job (for the algorithmic figures), read once
    d_ids = dev.malloc(tokens * TOPK * 4)
    rows_total, distinct_total = 0, 0
    src = job.d_x0
    for l in range(n_layers):
        dst = job.d_a if (l % 2 == 0) else job.d_b
        lb = job.base + l * job.slots_l * job.stride
        assert lib.q4_cuda_moe_layer_n(lb, job.stride, job.og, job.ou, job.od, N_EXPERT, src,
                                       job.d_norm + l * N_EMBD * 4, EPS, job.d_router + l * ROUTER_BYTES,
                                       N_EXPERT, TOPK, N_EMBD, N_FF, tokens, dst, d_ids, None, job.d_ws,
                                       job.ws)
        ids = dev.download(d_ids, (tokens, TOPK), np.int32)
        rows_total += ids.size + tokens
        distinct_total += len(np.unique(ids)) + 1
        if kind == "verify":
            src = dst
    hist = np.bincount(ids.ravel(), minlength=N_EXPERT)
    sampler = ClockSampler(local)
    sampler.start()
    ms, ms_e2e, launches = time_job(job, a.steps, warmup, lambda v: v)
    clocks = sampler.stop()
    err = lib.q4_cuda_device_error()
    if err:
        raise SystemExit("device error word %#x" % err)
    layers_per_step = n_layers if kind == "verify" else 1
    units = tokens * layers_per_step
    rows_step = rows_total / n_layers * layers_per_step
    distinct_step = distinct_total / n_layers * layers_per_step
    t = ms * 1e-3 / a.steps
    hbm, src_name = read_peaks()
    bytes_step = distinct_step * PACK + layers_per_step * ROUTER_BYTES
    ops_step = rows_step * 3 * N_EMBD * N_FF * 2.0
    peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(
        os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
    # the grouped product runs as 16-bit floating-point MMAs (the scales ride in the operands):
    # the denominator is the measured dense bf16 rate; the numerator counts each weight x
    # activation product once, although the kernel spends two MMAs on it (a two-term expansion)
    tc_peak = float(peaks.get("bf16_tflops", 1590.0))
    if kind == "prefill":
        roof = {"bound": "tensor", "achieved": ops_step / t / 1e12, "peak": tc_peak, "unit": "TFLOP/s",
                "frac": ops_step / t / 1e12 / tc_peak, "traffic": None,
                "peak_source": "measured bf16 burst" if peaks else "fallback bf16",
                "hbm_GBps": bytes_step / t / 1e9, "hbm_frac": bytes_step / t / 1e9 / hbm,
                "kernel": "whole step (%d launches)" % launches}
    else:
        roof = {"bound": "hbm", "achieved": bytes_step / t / 1e9, "peak": hbm, "unit": "GB/s",
                "frac": bytes_step / t / 1e9 / hbm, "traffic": None, "peak_source": src_name,
                "kernel": "whole step (%d launches)" % launches}
    name = ("config2: speculative-verify decode, 4 tokens x %d MoE layers per step" % n_layers
            if kind == "verify" else
            "config3: prefill chunk, 2048 tokens x 1 MoE layer per step, Zipf(1.1) expert skew "
            "(rows per expert max %d, median %d)" % (int(hist.max()), int(np.median(hist))))
    print(json.dumps({
        "metric": METRIC, "value": units / t, "unit": UNIT, "n_gpus": 1, "steps": a.steps, "warmup": warmup,
        "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 x IQ3_S, fp32 accumulate", "data": "synthetic",
        "config": {"workload": name, "l2": "inputs larger than L2: a step reads %.0f MB of weights"
                                          % (bytes_step / 1e6),
                   "routed_rows_per_step": rows_step, "distinct_experts_per_step": distinct_step,
                   "cuda_graph": bool(job.graph)},
        "clocks": clocks,
        "e2e": {"value": units * a.steps / (ms_e2e * 1e-3), "unit": UNIT,
                "h2d_bytes_per_step": job.nb, "d2h_bytes_per_step": job.nb},
        "gpu_launches": int(launches * a.steps * 2),
        "roofline": roof, "cpu_baseline": None}))


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
    ap.add_argument("--workload", default="auto", choices=["auto", "ep", "verify", "prefill"],
                    help="ep: the 64-token x 48-layer expert-parallel job (config 4) even on one GPU; "
                         "verify: 4 tokens x 48 layers (config 2); prefill: 2048 tokens x 1 layer (config 3)")
    a = ap.parse_args()
    rank, world, local = dist_setup(a.gpus)
    warmup = max(a.warmup, 3)
    if world > 1:       # one process per GPU: each sees only its own device
        os.environ["CUDA_VISIBLE_DEVICES"] = str(local)

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
                                 "kind": "reference", "cpu_model": cpu_model(),
                                 "sample": "%d steps x %d layer-tokens" % (steps, per_step)},
                "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if world == 1 and a.workload in ("verify", "prefill"):
        if a.steps == 2000 and a.warmup == 200:
            a.steps, warmup = 20, 3
        if a.layers == 48 and a.workload == "prefill":
            a.layers = 2
        run_batch(a, pkg, local, warmup, a.workload)
        return
    if world > 1 or a.workload == "ep":
        if a.steps == 2000 and a.warmup == 200:     # the single-layer defaults are too long here
            a.steps, warmup = 20, 3
        run_ep(a, pkg, rank, world, local, warmup)
        return

    wl = Workload(pkg, a.layers)
    lib = wl.lib
    launches0 = lib.q4_cuda_launch_count()
    # graphs of one pass over the layers each, plus one shorter graph for the remainder, so
    # that exactly `steps` steps are timed whatever the step count
    g_steps = min(a.layers, a.steps)
    wl.capture(g_steps)
    launches_per_step = (lib.q4_cuda_launch_count() - launches0) / (len(wl.graphs) * g_steps)
    n_graphs = a.steps // g_steps
    wl.capture_tail(a.steps % g_steps)
    wl.run_resident((warmup + g_steps - 1) // g_steps)
    wl.dev.sync()

    sampler = ClockSampler(local)
    sampler.start()
    # --- device-resident throughput ---
    wl.dev.sync()
    lib.q4_cuda_timer_begin()
    wl.run_resident(n_graphs, tail=True)
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
                     "frac": achieved / peak, "traffic": FUSED_DRAM_BYTES_PER_LAUNCH,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch "
                                       "(profiles/decode1_fused_kernel.md)",
                     "peak_source": peak_src,
                     "kernel": "whole step (%g launches/step)" % launches_per_step},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
