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
resident on the device (the K steps run as launches of the persistent kernel over
consecutive layers, y of a layer feeding the next); `e2e` goes through the
one-layer C-ABI call with the token's hidden state copied from pinned host memory
and the result read back every step.  Whatever K is, the timed set of steps is
repeated until at least 50 ms have been timed; the per-step time is the median
over the repeats.  `cpu_baseline` times the reference engine's own CPU path for
the same layer on this host's cores.  `details.other_workloads` carries the other
benchmark configurations (0, 2, 3 and 4 on one GPU), each with its own roofline
and CPU figure.  `--impl reference` prints the CPU arm alone.

N >= 2 (one process per GPU, torchrun environment): config 4, expert-parallel
decode of 64 tokens through 48 layers, strong scaling.
"""
import argparse
import faulthandler
import atexit
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

# CPU arm: the reference's expert pool gets the cores; its small host-side router GEMV (OpenMP in
# the reference's build) stays on one thread unless told otherwise -- an OpenMP team next to the
# pool's spinning workers was measured 13x slower (the line reports a figure with a passive team
# beside it).  Must be set before the OpenMP runtime is loaded.
os.environ.setdefault("OMP_NUM_THREADS", "1")

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
METRIC = "moe_layer_decode_tokens_per_s"
UNIT = "layer-tok/s"
DTYPE = "int8 x IQ3_S, fp32 accumulate"
MIN_TIMED_MS = 50.0
SEED = 2026
N_LAYERS = 48

CONFIG1 = {"workload": "config1: one MoE layer, decode batch 1, hidden 2048, ff 512, "
                       "512 experts top-10 + shared, IQ3_S x q8",
           "layers_rotated": N_LAYERS,
           "l2": "inputs larger than L2: every step reads a different layer (a repeat of the "
                 "timed steps reads at least 380 MB of weights)",
           "algorithmic_bytes_per_step": STEP_BYTES}


def config4(world, n_layers):
    return {"workload": "config4: expert-parallel decode, 64 tokens x %d MoE layers per step, 512 "
                        "experts top-10 + shared, experts sharded %d-way, one process per GPU"
                        % (n_layers, world),
            "l2": "inputs larger than L2: a step reads %d layers of weights" % n_layers,
            "tokens_per_rank": 64 // world, "experts_per_rank": N_EXPERT // world}


def read_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
        except Exception:
            pass
    return 6650.0, 1590.0, "fallback"


def read_traffic(name):
    """DRAM bytes per unit from the small JSON beside a profile summary (None if absent)."""
    p = os.path.join(ROOT, "profiles", name)
    try:
        return json.load(open(p))
    except Exception:
        return None


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


def cpu_model():
    try:
        for line in open("/proc/cpuinfo"):
            if line.startswith("model name"):
                return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


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


def median_step(lib, enqueue_set, units_per_set, warm_sets, min_ms=MIN_TIMED_MS, max_repeats=1000):
    """Device time per unit: `enqueue_set(r)` enqueues one set of steps (repeat number r); the
    set is repeated until min_ms have been timed, each repeat between its own pair of marks on
    the compute stream.  Returns (median ms per unit, repeats, total timed ms, launches)."""
    for r in range(warm_sets):
        enqueue_set(r)
    lib.q4_hip_stream_sync()
    # a first timed repeat sizes the run
    lib.q4_cuda_timer_mark(0)
    enqueue_set(warm_sets)
    lib.q4_cuda_timer_mark(1)
    first = max(lib.q4_cuda_timer_between_ms(0, 1), 1e-4)
    repeats = int(min(max_repeats, max(3, np.ceil(1.3 * min_ms / first))))   # the first set runs slow
    l0 = lib.q4_cuda_launch_count()
    for r in range(repeats):
        lib.q4_cuda_timer_mark(2 * r)
        enqueue_set(warm_sets + 1 + r)
        lib.q4_cuda_timer_mark(2 * r + 1)
    per = [lib.q4_cuda_timer_between_ms(2 * r, 2 * r + 1) for r in range(repeats)]
    launches = lib.q4_cuda_launch_count() - l0
    return float(np.median(per)) / units_per_set, repeats, float(np.sum(per)), int(launches)


def median_wall(run_set, units_per_set, warm_sets, min_ms=MIN_TIMED_MS, max_repeats=1000):
    """Wall-clock time per unit of a host-synchronous set of steps, median over repeats."""
    for r in range(warm_sets):
        run_set(r)
    t0 = time.perf_counter()
    run_set(warm_sets)
    first = max(1e3 * (time.perf_counter() - t0), 1e-3)
    repeats = int(min(max_repeats, max(3, np.ceil(min_ms / first))))
    per = []
    for r in range(repeats):
        t0 = time.perf_counter()
        run_set(warm_sets + 1 + r)
        per.append(1e3 * (time.perf_counter() - t0))
    return float(np.median(per)) / units_per_set, repeats


class StackDesc(ctypes.Structure):
    _fields_ = [("base", ctypes.c_void_p), ("norm", ctypes.c_void_p), ("router", ctypes.c_void_p)]


class Model:
    """n_layers MoE layers of seeded synthetic weights generated on the device: an arena of
    n_layers x (experts_here + 1) packs (the shared expert last in each layer), fp32 routers
    and norm weights.  Expert (layer, e) has the same bytes whatever shard holds it: a rank
    of an expert-parallel run generates its range [e_first, e_first + e_count) of the full
    seeded tensor."""

    def __init__(self, dev, n_layers, arena=0, e_first=0, e_count=N_EXPERT, seed=SEED):
        self.dev, self.lib = dev, dev.lib
        lib = self.lib
        self.n_layers, self.arena, self.e_count = n_layers, arena, e_count
        self.slots_l = e_count + 1
        bpp = PACK // IQ3S_BLOCK            # super-blocks per expert pack
        if not lib.q4_hip_experts_alloc_a(arena, n_layers * self.slots_l, PACK):
            raise MemoryError("expert arena of %d slots" % (n_layers * self.slots_l))
        self.base, self.stride = lib.q4_hip_experts_base_a(arena), lib.q4_hip_experts_stride_a(arena)
        for l in range(n_layers):
            lb = self.layer_base(l)
            assert lib.q4_cuda_synth_iq3s_at(lb, e_count * bpp, seed, (l * (N_EXPERT + 1) + e_first) * bpp)
            assert lib.q4_cuda_synth_iq3s_at(lb + e_count * self.stride, bpp, seed,
                                             (l * (N_EXPERT + 1) + N_EXPERT) * bpp)
        self.tiled = bool(lib.q4_cuda_experts_tiled_a(arena))
        if self.tiled:      # generated in the engine's byte order: convert to the resident format
            assert lib.q4_cuda_experts_retile_a(arena, 0, n_layers * self.slots_l)
        self.d_router = dev.malloc(n_layers * ROUTER_BYTES)
        assert lib.q4_cuda_synth_normal(self.d_router, n_layers * N_EXPERT * N_EMBD, seed + 1, 0.0, 0.02)
        self.d_norm = dev.malloc(n_layers * N_EMBD * 4)
        assert lib.q4_cuda_synth_normal(self.d_norm, n_layers * N_EMBD, seed + 2, 1.0, 0.1)
        rb = N_EMBD // 256 * IQ3S_BLOCK
        self.og, self.ou, self.od = 0, N_FF * rb, 2 * N_FF * rb
        dev.sync()

    def layer_base(self, l):
        return self.base + l * self.slots_l * self.stride

    def router(self, l):
        return self.d_router + l * ROUTER_BYTES

    def norm(self, l):
        return self.d_norm + l * N_EMBD * 4

    def zipf_skew(self, pkg, x_all):
        """Expert popularity skewed by a Zipf(1.1) bias on the router logits: every token carries
        the same value A in coordinate 0 (norm weight 1 there), and router column 0 holds
        bias_e / (normalised A), so logit_e = N(0, ~1) + bias_e."""
        A = 4.0
        x_all[:, 0] = A
        xn0 = A / np.sqrt((A * A + N_EMBD - 1.0) / N_EMBD)
        col = (pkg.synth.zipf_bias(N_EXPERT, 1.1) / xn0).astype(np.float32)
        one = np.ones(1, np.float32)
        self.dev.sync()
        for l in range(self.n_layers):
            r = self.dev.download(self.router(l), (N_EXPERT, N_EMBD), np.float32)
            r[:, 0] = col
            self.dev.write(self.router(l), r)
            self.dev.write(self.norm(l), one)

    def host_layers(self, layers):
        """Copies of some layers' tensors on the host, engine byte order (for the CPU arm)."""
        assert self.e_count == N_EXPERT
        out = []
        for l in layers:
            packs = np.empty((self.slots_l, PACK), np.uint8)
            for e in range(self.slots_l):
                assert self.lib.q4_cuda_experts_get_a(self.arena, l * self.slots_l + e, packs[e].ctypes.data, PACK)
            out.append({
                "experts": packs[:N_EXPERT], "shared": packs[N_EXPERT],
                "router": self.dev.download(self.router(l), (N_EXPERT, N_EMBD), np.float32),
                "norm_w": self.dev.download(self.norm(l), (N_EMBD,), np.float32)})
        return out

    def release(self):
        self.lib.q4_hip_experts_free_a(self.arena)
        self.dev.free(self.d_router)
        self.dev.free(self.d_norm)


class Decode1:
    """Config 1 on a Model: one token, one layer per step."""

    def __init__(self, pkg, model):
        self.pkg, self.m, self.dev, self.lib = pkg, model, model.dev, model.lib
        lib, dev = self.lib, self.dev
        self.n_x = 64
        self.x_host = pkg.synth.hidden(SEED + 3, self.n_x, N_EMBD)
        self.d_xpool = dev.upload(self.x_host)
        self.d_y = dev.malloc(N_EMBD * 4)
        self.h_x = lib.q4_hip_host_alloc_coh(N_EMBD * 4)
        self.h_y = lib.q4_hip_host_alloc_coh(N_EMBD * 4)
        self.y_out = np.zeros(N_EMBD, np.float32)
        self.stack_plans = {}
        self.plans = None

    def stack_plan(self, first, count):
        """The persistent kernel over layers first, first + 1, ... (mod the model's layers)."""
        key = (first, count)
        if key not in self.stack_plans:
            m = self.m
            arr = (StackDesc * count)()
            for i in range(count):
                l = (first + i) % m.n_layers
                arr[i].base, arr[i].norm, arr[i].router = m.layer_base(l), m.norm(l), m.router(l)
            p = self.lib.q4_cuda_decode_stack_plan(arr, count, m.stride, m.og, m.ou, m.od, N_EXPERT, EPS,
                                                   N_EXPERT, TOPK, N_EMBD, N_FF)
            if not p:
                raise RuntimeError("q4_cuda_decode_stack_plan refused")
            self.stack_plans[key] = p
        return self.stack_plans[key]

    def enqueue_steps(self, k, r):
        """k consecutive layer-steps of one token (repeat number r picks the token and the first
        layer), as launches of at most 48 layers each; y of a layer is x of the next."""
        m = self.m
        first = (r * k) % m.n_layers
        x = self.d_xpool + (r % self.n_x) * N_EMBD * 4
        done = 0
        while done < k:
            n = min(m.n_layers, k - done)
            if not self.lib.q4_cuda_decode_stack_dev(self.stack_plan((first + done) % m.n_layers, n), x, self.d_y,
                                                     None, None):
                raise RuntimeError("q4_cuda_decode_stack_dev refused")
            x = self.d_y    # the next launch continues from this one's output (same buffer: read at
            done += n       # the start of the launch, written at its end)

    def e2e_steps(self, k, r):
        """k steps through the one-layer host-buffer call: the token's row is written into pinned
        host memory, the layer runs, the 8 KB result is read on the host -- every step."""
        lib, m = self.lib, self.m
        if self.plans is None:
            self.plans = []
            for l in range(m.n_layers):
                p = lib.q4_cuda_decode_plan(m.layer_base(l), m.stride, m.og, m.ou, m.od, N_EXPERT, m.norm(l), EPS,
                                            m.router(l), N_EXPERT, TOPK, N_EMBD, N_FF)
                if not p:
                    raise RuntimeError("q4_cuda_decode_plan refused")
                self.plans.append(p)
        run, h_y = lib.q4_cuda_decode_plan_host, self.h_y
        xp = [self.x_host[i].ctypes.data for i in range(self.n_x)]      # the call copies the row itself
        y_out, nb = self.y_out.ctypes.data, N_EMBD * 4
        for i in range(r * k, r * k + k):
            if not run(self.plans[i % m.n_layers], xp[i % self.n_x], h_y):
                raise RuntimeError("q4_cuda_decode_plan_host refused")
            ctypes.memmove(y_out, h_y, nb)

    def e2e_stack(self, r):
        """One token through all layers in one host-buffer call (row in, row out)."""
        ctypes.memmove(self.h_x, self.x_host[r % self.n_x].ctypes.data, N_EMBD * 4)
        if not self.lib.q4_cuda_decode_stack_host(self.stack_plan(0, self.m.n_layers), self.h_x, self.h_y):
            raise RuntimeError("q4_cuda_decode_stack_host refused")
        ctypes.memmove(self.y_out.ctypes.data, self.h_y, N_EMBD * 4)

    def session_begin(self):
        """The resident form of the same kernel: one launch, then one doorbell ring per step; step s runs
        layer s mod n_layers of the model."""
        self.ses = self.lib.q4_cuda_decode_session_begin(self.stack_plan(0, self.m.n_layers), 1, 0, 0)
        if not self.ses:
            raise RuntimeError("q4_cuda_decode_session_begin refused")
        self.x_ptrs = [self.x_host[i].ctypes.data for i in range(self.n_x)]

    def session_steps(self, k, r):
        """k steps of the session: the token's row goes from host memory into the kernel, the layer's
        8 KB result comes back into host memory -- every step."""
        step, ses, y, xp, n = self.lib.q4_cuda_decode_session_step, self.ses, self.y_out.ctypes.data, self.x_ptrs, self.n_x
        for i in range(r * k, r * k + k):
            if not step(ses, xp[i % n], y):
                raise RuntimeError("q4_cuda_decode_session_step failed")

    def session_end(self):
        if getattr(self, "ses", None):
            self.lib.q4_cuda_decode_session_end(self.ses)
            self.ses = None

    def release(self):
        self.session_end()
        for p in self.stack_plans.values():
            self.lib.q4_cuda_decode_stack_free(p)
        for p in self.plans or []:
            self.lib.q4_cuda_decode_plan_free(p)
        self.stack_plans, self.plans = {}, None
        self.lib.q4_hip_host_free_coh(self.h_x)
        self.lib.q4_hip_host_free_coh(self.h_y)


EP_TOKENS = 64          # config 4: batch of 64 tokens ...


class BatchJob:
    """`tokens` tokens through the layers of a Model, y of a layer feeding the next (chain) or
    every layer on the same input rows; this object is one rank's part (world == 1: the whole
    job on one GPU through q4_cuda_moe_layer_n)."""

    def __init__(self, pkg, model, ep, rank, world, tokens, layers, chain=True, x_all=None, form="ar"):
        self.pkg, self.m, self.dev, self.lib = pkg, model, model.dev, model.lib
        lib, dev = self.lib, self.dev
        self.ep, self.world, self.layers, self.chain = ep, world, list(layers), chain
        self.tokens = tokens
        self.t_local = tokens // world
        if x_all is None:
            x_all = pkg.synth.hidden(SEED + 3, tokens, N_EMBD)
        # expert-parallel forms: "ar" keeps all token rows on every rank and sums the ranks' partial
        # rows with one all-reduce per layer; "a2a" keeps a rank's own tokens only and exchanges
        # twice per layer (gather of rows and picks, all-to-all of partial rows)
        self.form = form
        self.rows = tokens if (world > 1 and form == "ar") else self.t_local
        first = 0 if self.rows == tokens else rank * self.t_local
        self.x_host = np.ascontiguousarray(x_all[first:first + self.rows])
        self.nb = nb = self.rows * N_EMBD * 4
        self.d_x0, self.d_a, self.d_b = dev.upload(self.x_host), dev.malloc(nb), dev.malloc(nb)
        self.h_x, self.h_y = lib.q4_hip_host_alloc_coh(nb), lib.q4_hip_host_alloc_coh(nb)
        ctypes.memmove(self.h_x, self.x_host.ctypes.data, nb)
        if world == 1:
            self.ws = lib.q4_cuda_moe_layer_n_ws_bytes(self.t_local, TOPK, N_EXPERT, N_EMBD, N_FF)
        else:
            self.ws = ep.q4_cuda_ep_layer_ws_bytes(world, self.t_local, TOPK, N_EXPERT, N_EMBD, N_FF)
        self.d_ws = dev.malloc(self.ws)
        self.graph = None
        self.d_out = self.d_a
        self.one_per_step = False   # a step is ONE layer, the layers taken in turn (no chaining)
        self.turn = 0

    def layer(self, l, src, dst, d_ids=None):
        m = self.m
        if self.world == 1:
            ok = self.lib.q4_cuda_moe_layer_n(m.layer_base(l), m.stride, m.og, m.ou, m.od, N_EXPERT, src, m.norm(l),
                                              EPS, m.router(l), N_EXPERT, TOPK, N_EMBD, N_FF, self.t_local, dst,
                                              d_ids, None, self.d_ws, self.ws)
        else:
            call = self.ep.q4_cuda_ep_layer_ar if self.form == "ar" else self.ep.q4_cuda_ep_layer
            ok = call(m.layer_base(l), m.stride, m.og, m.ou, m.od, 1, src, m.norm(l), EPS, m.router(l), N_EXPERT,
                      TOPK, N_EMBD, N_FF, self.t_local, dst, self.d_ws, self.ws)
        if not ok:
            raise RuntimeError("layer call refused")

    def enqueue(self, layers=None):
        if self.one_per_step:
            self.layer(self.layers[self.turn % len(self.layers)], self.d_x0, self.d_a)
            self.turn += 1
            self.d_out = self.d_a
            return
        src = self.d_x0
        for i, l in enumerate(layers if layers is not None else self.layers):
            dst = self.d_a if (i % 2 == 0) else self.d_b
            self.layer(l, src, dst)
            if self.chain:
                src = dst
        self.d_out = dst

    def routing_stats(self):
        """(routed rows incl. shared, distinct experts incl. shared, last layer's histogram),
        summed over the job's layers, read once from the device."""
        assert self.world == 1
        d_ids = self.dev.malloc(self.tokens * TOPK * 4)
        rows, distinct, src, hist = 0, 0, self.d_x0, None
        for i, l in enumerate(self.layers):
            dst = self.d_a if (i % 2 == 0) else self.d_b
            self.layer(l, src, dst, d_ids)
            ids = self.dev.download(d_ids, (self.tokens, TOPK), np.int32)
            rows += ids.size + self.tokens
            distinct += len(np.unique(ids)) + 1
            hist = np.bincount(ids.ravel(), minlength=N_EXPERT)
            if self.chain:
                src = dst
        self.dev.free(d_ids)
        return rows, distinct, hist

    def try_capture(self):
        """One CUDA graph per step; plain launches if the capture is refused (e.g. by the
        collective library)."""
        if self.one_per_step or self.lib.q4_hip_graph_begin() != 1:
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

    def output(self):
        return self.dev.download(self.d_out, (self.rows, N_EMBD), np.float32)

    def release(self):
        if self.graph:      # a graph that holds collective nodes must go before the communicator does
            self.lib.q4_hip_graph_free(self.graph)
            self.graph = None
        for p in (self.d_x0, self.d_a, self.d_b, self.d_ws):
            self.dev.free(p)
        self.lib.q4_hip_host_free_coh(self.h_x)
        self.lib.q4_hip_host_free_coh(self.h_y)


def time_job(job, steps, warmup, barrier_max, min_ms=MIN_TIMED_MS):
    """(median ms per step resident, median ms per step end to end, launches per step, repeats)
    for sets of `steps` steps, max over ranks."""
    lib = job.lib
    l0 = lib.q4_cuda_launch_count()
    job.enqueue()
    job.dev.sync()
    launches = lib.q4_cuda_launch_count() - l0
    job.try_capture()
    for _ in range(max(warmup, 3)):
        job.step()
    job.dev.sync()
    # size the run on a first timed set (the same count on every rank)
    barrier_max(0.0)
    lib.q4_cuda_timer_mark(0)
    for _ in range(steps):
        job.step()
    lib.q4_cuda_timer_mark(1)
    first = barrier_max(max(lib.q4_cuda_timer_between_ms(0, 1), 1e-3))
    repeats = int(min(500, max(3, np.ceil(1.3 * min_ms / first))))
    per = []
    for r in range(repeats):
        barrier_max(0.0)
        lib.q4_cuda_timer_mark(0)
        for _ in range(steps):
            job.step()
        lib.q4_cuda_timer_mark(1)
        per.append(barrier_max(lib.q4_cuda_timer_between_ms(0, 1)))
    ms = float(np.median(per)) / steps
    job.dev.sync()
    for _ in range(2):
        job.step_e2e()
    per = []
    for r in range(max(3, min(repeats, int(np.ceil(min_ms / (ms * steps))) + 1))):
        barrier_max(0.0)
        t0 = time.perf_counter()
        for _ in range(steps):
            job.step_e2e()
        per.append(barrier_max(1e3 * (time.perf_counter() - t0)))
    ms_e2e = float(np.median(per)) / steps
    return ms, ms_e2e, launches, repeats


# ------------------------------------------------------------------ CPU arms (the reference's own code)

def ref_lib():
    from oracle import pyoracle
    ref = pyoracle.reference()
    if ref is not None:
        ncpu = os.cpu_count() or 2
        os.environ.setdefault("Q4_CPU_THREADS", str(max(1, min(16, ncpu - 1))))
    return ref


def cpu_layers_tokens(ref, layers, x, n_tok, budget_s, chain=True):
    """Times layer jobs of n_tok tokens each on the reference's CPU path for about budget_s
    seconds: host-side norm + fp32 router + softmax/top-k per token, expert work on its worker
    pool (one-token jobs for n_tok == 1, window jobs otherwise).  Returns the baseline dict."""
    x = np.ascontiguousarray(x[:n_tok])
    t, _, _ = ref.time_layers_win(layers, TOPK, 2, x, N_EMBD, N_FF, chain, EPS)     # warm-up, pool start
    per = max(t / 2, 1e-5)
    steps = int(max(4, min(20000, budget_s / per)))
    t, t_router, _ = ref.time_layers_win(layers, TOPK, steps, x, N_EMBD, N_FF, chain, EPS)
    lt = steps * n_tok
    return {"value": lt / t, "unit": UNIT, "cores": ref.threads(), "kind": "reference", "cpu_model": cpu_model(),
            "sample": "%d layer jobs of %d token(s) over %d layers of weights (%.1f s): norm, router, top-k on "
                      "the host, experts on the reference's worker pool (%s)"
                      % (steps, n_tok, len(layers), t, "q4_cpuex_dispatch2" if n_tok == 1 else
                         "q4_cpuex_dispatch_win, windows of up to %d tokens" % min(8, 64 // (TOPK + 1))),
            "ms_per_step": 1e3 * t / lt, "router_ms": 1e3 * t_router / lt,
            "experts_ms": 1e3 * (t - t_router) / lt, "omp_threads": int(os.environ.get("OMP_NUM_THREADS", "1"))}


# Every CPU leg runs in a child process.  The reference's worker pool is its own code, run unmodified,
# and a run of small jobs has been seen not to return from it (about one default run in three hung in
# the one-expert jobs of config 0); a child can be given a time limit and tried again, the parent cannot.
_CPU_DIRS = []


def _cpu_dir():
    import shutil
    import tempfile
    base = "/dev/shm" if os.path.isdir("/dev/shm") and shutil.disk_usage("/dev/shm").free > (4 << 30) else None
    d = tempfile.mkdtemp(prefix="q4b_cpu_", dir=base)
    _CPU_DIRS.append(d)
    atexit.register(shutil.rmtree, d, True)
    return d


def dump_layers(layers):
    """The layers' tensors as .npy files a child maps (two layers: 1.4 GB); returns the directory."""
    d = _cpu_dir()
    for i, L in enumerate(layers):
        for k in ("experts", "shared", "router", "norm_w"):
            np.save(os.path.join(d, "l%d_%s.npy" % (i, k)), np.ascontiguousarray(L[k]))
    return d


def load_layers(d):
    out, i = [], 0
    while os.path.exists(os.path.join(d, "l%d_experts.npy" % i)):
        out.append({k: np.load(os.path.join(d, "l%d_%s.npy" % (i, k)), mmap_mode="r")
                    for k in ("experts", "shared", "router", "norm_w")})
        i += 1
    return out


def cpu_child(kind, seconds, layers_dir=None, x=None, n_tok=1, chain=True, env=None, extra=()):
    """One CPU leg in a child: kind 'layers' (cpu_layers_tokens), 'config0' (cpu_config0) or 'arm'
    (the --impl reference loop).  Weights from layers_dir, else generated on the host.  Returns the
    child's JSON object, or {"unavailable": why} after two attempts."""
    cmd = [sys.executable, os.path.abspath(__file__), "--cpu-probe", "--cpu-kind", kind, "--cpu-seconds",
           str(seconds), "--cpu-tokens", str(n_tok)] + list(extra)
    if not chain:
        cmd.append("--cpu-nochain")
    if layers_dir:
        cmd += ["--cpu-dir", layers_dir]
        if x is not None:
            np.save(os.path.join(layers_dir, "x.npy"), np.ascontiguousarray(x, np.float32))
    limit = 120 + 8 * float(seconds)
    why = "not run"
    for _ in (1, 2):
        try:
            r = subprocess.run(cmd, env=env or os.environ, capture_output=True, text=True, timeout=limit)
            lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
            if lines:
                return json.loads(lines[-1])
            why = "child exited %d: %s" % (r.returncode, r.stderr.strip()[-300:])
        except subprocess.TimeoutExpired:
            why = "the reference's worker pool did not return within %d s (tried twice)" % limit
    return {"unavailable": why}


def cpu_probe_main(a):
    """The child: one CPU leg, one JSON object on stdout."""
    pkg = entry.load_package()
    ref = ref_lib()
    if ref is None:
        print(json.dumps({"unavailable": "compiled reference CPU path (oracle/_ref) not present"}))
        return
    if a.cpu_dir:
        layers = load_layers(a.cpu_dir)
        xp = os.path.join(a.cpu_dir, "x.npy")
        x = np.load(xp) if os.path.exists(xp) else pkg.synth.hidden(7, 64, N_EMBD)
    else:
        layers = [pkg.synth.layer(SEED + 17 * l, N_EXPERT, N_EMBD, N_FF) for l in range(2)]
        x = pkg.synth.hidden(7, 64, N_EMBD)
    if a.cpu_kind == "config0":
        d = cpu_config0(ref, layers[0], x, a.cpu_seconds)
    elif a.cpu_kind == "arm":
        # the --impl reference loop: warm-up, then `steps` timed samples of `jobs` layer jobs each
        xs = x[:a.cpu_tokens]
        ref.time_layers_win(layers, TOPK, 2, xs, N_EMBD, N_FF, True, EPS)
        for _ in range(a.cpu_warm):
            ref.time_layers_win(layers, TOPK, a.cpu_jobs, xs, N_EMBD, N_FF, True, EPS)
        t = t_router = 0.0
        for _ in range(a.cpu_steps):
            dt, dr, _y = ref.time_layers_win(layers, TOPK, a.cpu_jobs, xs, N_EMBD, N_FF, True, EPS)
            t += dt
            t_router += dr
        d = {"t": t, "t_router": t_router, "cores": ref.threads(), "cpu_model": cpu_model(),
             "omp_threads": int(os.environ.get("OMP_NUM_THREADS", "1"))}
    else:
        d = cpu_layers_tokens(ref, layers, x, a.cpu_tokens, a.cpu_seconds, chain=not a.cpu_nochain)
    print(json.dumps(d))


def cpu_probe_passive_omp(seconds):
    """The config-1 CPU arm with a small passive OpenMP team for the router product (the default
    arm keeps it on one thread), so that choice is visible in numbers; host-generated weights."""
    d = cpu_child("layers", seconds, env=dict(os.environ, OMP_NUM_THREADS="4", OMP_WAIT_POLICY="passive"))
    if "unavailable" not in d:
        d = {k: d[k] for k in ("value", "ms_per_step", "router_ms", "experts_ms", "cores", "omp_threads")}
        d["omp_wait_policy"] = "passive"
    return d


def cpu_config0(ref, layer, x, budget_s):
    """Config 0 on the CPU path: one expert, one token per job, distinct experts back to back."""
    packs = [layer["experts"][e] for e in range(N_EXPERT)]
    jobs = 256
    ids = (np.arange(jobs, dtype=np.int32) % N_EXPERT).reshape(jobs, 1)
    wts = np.ones((jobs, 1), np.float32)
    t = ref.time_jobs(packs, ids, wts, 1, x, N_EMBD, N_FF)
    reps = int(max(1, min(200, budget_s / max(t, 1e-4))))
    ids = np.tile(ids, (reps, 1))
    wts = np.tile(wts, (reps, 1))
    t = ref.time_jobs(packs, ids, wts, 1, x, N_EMBD, N_FF)
    n = jobs * reps
    return {"value": n / t, "unit": "expert-tok/s", "cores": ref.threads(), "kind": "reference",
            "cpu_model": cpu_model(), "sample": "%d one-expert jobs over 512 distinct experts (%.1f s), "
            "q4_cpuex_dispatch2 with k = 1" % (n, t), "ms_per_step": 1e3 * t / n}


# ------------------------------------------------------------------ the other configurations on one GPU

def roof_hbm(bytes_per_step, t_step, kernel):
    hbm, _, src = read_peaks()
    ach = bytes_per_step / t_step / 1e9
    return {"bound": "hbm", "achieved": ach, "peak": hbm, "unit": "GB/s", "frac": ach / hbm, "traffic": None,
            "peak_source": src, "kernel": kernel}


def measure_config0(pkg, model, ref_layer=None, cpu_s=0.0):
    """Config 0: ONE expert's feed-forward for one token per unit, 512 distinct experts back to
    back (q4_hip_moe_exec_dev with a one-entry list; a CUDA graph of 512 calls per set)."""
    dev, lib = model.dev, model.lib
    n = N_EXPERT
    x = pkg.synth.hidden(SEED + 5, 1, N_EMBD)[0]
    d_x, d_y, d_h = dev.upload(x), dev.malloc(N_EMBD * 4), dev.malloc(N_FF * 4)
    d_es = dev.upload(np.arange(n, dtype=np.int32))
    d_ew = dev.upload(np.ones(n, np.float32))
    d_one = dev.upload(np.array([1], np.int32))
    lib.q4_hip_fill(d_y, 0.0, N_EMBD)

    def call(e, layer):
        if not lib.q4_hip_moe_exec_dev(model.layer_base(layer), model.stride, d_es + 4 * e, d_ew + 4 * e, d_one, 21,
                                       model.og, 21, model.ou, 21, model.od, d_x, d_h, None, None, d_y, N_FF,
                                       N_EMBD, N_EMBD):
            raise RuntimeError("q4_hip_moe_exec_dev refused")
    graphs = []
    for layer in range(min(2, model.n_layers)):      # two layers in turn: 1.4 GB between reuses
        assert lib.q4_hip_graph_begin() == 1
        for e in range(n):
            call(e, layer)
        g = lib.q4_hip_graph_end()
        if not g:
            raise RuntimeError("graph capture failed")
        graphs.append(g)
    ms, repeats, _, launches = median_step(
        lib, lambda r: lib.q4_hip_graph_launch(graphs[r % len(graphs)]) or None, n, 2)
    # end to end: the token's row goes up, one expert runs, the 8 KB result comes back, per unit
    h_x, h_y = lib.q4_hip_host_alloc_coh(N_EMBD * 4), lib.q4_hip_host_alloc_coh(N_EMBD * 4)
    ctypes.memmove(h_x, x.ctypes.data, N_EMBD * 4)
    es = np.arange(n, dtype=np.int32)
    one = np.ones(1, np.float32)

    def e2e_set(r):
        for e in range(64):
            lib.q4_hip_h2d_async(d_x, h_x, N_EMBD * 4)
            lib.q4_hip_fill(d_y, 0.0, N_EMBD)
            if not lib.q4_hip_moe_exec(model.layer_base(r % 2), model.stride, es[e:].ctypes.data, one.ctypes.data, 1,
                                       21, model.og, 21, model.ou, 21, model.od, d_x, d_h, None, None, d_y, N_FF,
                                       N_EMBD, N_EMBD):
                raise RuntimeError("q4_hip_moe_exec refused")
            lib.q4_hip_d2h_async(h_y, d_y, N_EMBD * 4)
            lib.q4_hip_stream_sync()
    ms_e2e, _ = median_wall(e2e_set, 64, 1)
    for g in graphs:
        lib.q4_hip_graph_free(g)
    for p in (d_x, d_y, d_h, d_es, d_ew, d_one):
        dev.free(p)
    lib.q4_hip_host_free_coh(h_x)
    lib.q4_hip_host_free_coh(h_y)
    entry_ = {"workload": "config0: one IQ3_S expert feed-forward (gate, up, SwiGLU, down), one token per unit, "
                          "512 distinct experts back to back",
              "value": 1e3 / ms, "unit": "expert-tok/s", "ms_per_step": ms, "repeats": repeats,
              "gpu_launches_per_unit": launches / (repeats * n),
              "e2e": {"value": 1e3 / ms_e2e, "unit": "expert-tok/s", "h2d_bytes_per_step": N_EMBD * 4,
                      "d2h_bytes_per_step": N_EMBD * 4},
              "roofline": roof_hbm(PACK, ms * 1e-3, "whole unit (launch chain)"), "cpu_baseline": None}
    if ref_layer is not None and cpu_s > 0:     # ref_layer: the directory of the dumped layers
        entry_["cpu_baseline"] = cpu_child("config0", cpu_s, ref_layer, pkg.synth.hidden(7, 64, N_EMBD))
    return entry_


def measure_batch(pkg, model, kind, steps, warmup, cpu_layers=None, cpu_s=0.0):
    """verify  (config 2): 4 tokens (1 + 3 drafts) through 48 layers per step, y of a layer feeding the next.
    prefill (config 3): 2048 tokens through one layer per step, expert popularity skewed by Zipf(1.1);
                        consecutive steps alternate between two layers of weights.
    ep1     (config 4 on one GPU): 64 tokens through 48 layers per step."""
    if kind == "verify":
        tokens, layers, name = 4, range(model.n_layers), \
            "config2: speculative-verify decode, 4 tokens x %d MoE layers per step" % model.n_layers
    elif kind == "ep1":
        tokens, layers, name = EP_TOKENS, range(model.n_layers), config4(1, model.n_layers)["workload"]
    else:
        tokens, layers, name = 2048, range(model.n_layers), None
    x_all = pkg.synth.hidden(SEED + 3, tokens, N_EMBD)
    if kind == "prefill":
        model.zipf_skew(pkg, x_all)
    job = BatchJob(pkg, model, None, 0, 1, tokens, layers, chain=(kind != "prefill"), x_all=x_all)
    rows, distinct, hist = job.routing_stats()
    n_l = len(job.layers)
    if kind == "prefill":
        job.one_per_step = True
        name = ("config3: prefill chunk, 2048 tokens x 1 MoE layer per step, Zipf(1.1) expert skew "
                "(rows per expert max %d, median %d)" % (int(hist.max()), int(np.median(hist))))
    layers_per_step = 1 if kind == "prefill" else n_l
    ms, ms_e2e, launches, repeats = time_job(job, steps, warmup, lambda v: v)
    err = job.lib.q4_cuda_device_error()
    if err:
        raise SystemExit("device error word %#x" % err)
    units = tokens * layers_per_step
    rows_step = rows / n_l * layers_per_step
    distinct_step = distinct / n_l * layers_per_step
    t = ms * 1e-3
    hbm, tc_peak, src = read_peaks()
    bytes_step = distinct_step * PACK + layers_per_step * ROUTER_BYTES
    if kind == "prefill":
        # the grouped product runs as 16-bit floating-point MMAs (the scales ride in the operands):
        # the denominator is the measured dense bf16 rate; the numerator counts each weight x
        # activation product once, although the kernel spends two MMAs on it (a two-term expansion)
        ops_step = rows_step * 3 * N_EMBD * N_FF * 2.0
        roof = {"bound": "tensor", "achieved": ops_step / t / 1e12, "peak": tc_peak, "unit": "TFLOP/s",
                "frac": ops_step / t / 1e12 / tc_peak, "traffic": None, "peak_source": src + " bf16 burst",
                "hbm_GBps": bytes_step / t / 1e9, "hbm_frac": bytes_step / t / 1e9 / hbm,
                "kernel": "whole step (%d launches)" % launches}
    else:
        roof = roof_hbm(bytes_step, t, "whole step (%d launches)" % launches)
    out = {"workload": name, "value": units / t, "unit": UNIT, "ms_per_step": ms, "steps": steps,
           "repeats": repeats, "tokens_per_step": tokens, "layers_per_step": layers_per_step,
           "routed_rows_per_step": rows_step, "distinct_experts_per_step": distinct_step,
           "cuda_graph": bool(job.graph), "gpu_launches_per_step": launches,
           "e2e": {"value": units / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": job.nb,
                   "d2h_bytes_per_step": job.nb},
           "roofline": roof, "cpu_baseline": None}
    if kind == "prefill" and cpu_s > 0:     # the skewed routers
        cpu_layers = dump_layers(model.host_layers(range(min(2, model.n_layers))))
    if cpu_layers is not None and cpu_s > 0:    # cpu_layers: the directory of the dumped layers
        n_tok = min(tokens, 64 if kind != "prefill" else 160)
        cb = cpu_child("layers", cpu_s, cpu_layers, x_all[:n_tok], n_tok, chain=(kind != "prefill"))
        if n_tok != tokens and "sample" in cb:
            cb["sample"] += "; %d of the step's %d tokens" % (n_tok, tokens)
        out["cpu_baseline"] = cb
    job.release()
    return out


# ------------------------------------------------------------------ config 4 on N GPUs

def ep_roofline(world, n_layers, t_step):
    """HBM roofline of the expert-parallel job over all ranks: every rank reads the router of
    each layer and the packs of the distinct experts routed to it plus its copy of the shared
    expert.  The number of distinct routed experts per layer is the expectation for uniform
    routing, E * (1 - (1 - k/E)^T) = 367 of 512 at 64 tokens, not a count of this run."""
    hbm, _, src = read_peaks()
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
    same job alone on its GPU: the line carries its own 1-GPU reference, the speed-up against
    it, and the difference between the two results for the tokens rank 0 owns."""
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

    n_layers = a.layers if a.layers else N_LAYERS
    e_local = N_EXPERT // world
    model = Model(dev, n_layers, 0, rank * e_local, e_local)
    job = BatchJob(pkg, model, ep, rank, world, EP_TOKENS, range(n_layers))
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms, ms_e2e, launches, repeats = time_job(job, a.steps, warmup, barrier_max)
    clocks = sampler.stop() if rank == 0 else None
    graphed = bool(job.graph)
    err = lib.q4_cuda_device_error()
    if err:
        raise SystemExit("device error word %#x" % err)
    floor = None
    if ep is not None:
        f2 = (ctypes.c_float * 2)()
        if ep.q4_cuda_ep_exchange_floor_us(job.t_local, N_EMBD, TOPK, N_EXPERT, N_FF, job.d_ws, job.ws, 50, f2):
            floor = {"gather_plus_all_to_all": barrier_max(f2[0]), "all_reduce": barrier_max(f2[1]),
                     "what": "one layer's collectives alone, with the layer's payload sizes, microseconds"}
    # results for the comparison with one GPU: the first layer alone (every rank takes part in its
    # exchanges), and the whole stack
    job.enqueue(layers=[0])
    dev.sync()
    y_ep_l0 = job.output() if rank == 0 else None
    job.step()
    dev.sync()
    y_ep = job.output() if rank == 0 else None
    details = {"cuda_graph": graphed, "repeats": repeats, "exchange_floor_us": floor,
               "form": "every rank holds all 64 token rows; one all-reduce of the partial rows per layer"}
    if ep is not None:
        e2 = ep.q4_cuda_ep_error()
        if e2:
            raise SystemExit("expert-parallel error word %#x" % e2)
        own = ep.q4_cuda_ep_allreduce_mode(2) == 1
        details["all_reduce"] = ("ep_allreduce_k: the library's kernel over IPC-mapped peer memory" if own
                                 else "ncclAllReduce (the ranks' buffers could not be mapped through CUDA IPC)")
        # variants of the same job, for comparison: ncclAllReduce instead of the library's kernel, and the
        # routing split over the ranks with a peer gather of the picks
        variants = {}
        if own:
            for name, ar, split in (("nccl_all_reduce", 0, 0), ("split_routing", 2, 1)):
                ep.q4_cuda_ep_allreduce_mode(ar)
                ep.q4_cuda_ep_split_routing(split)
                job_n = BatchJob(pkg, model, ep, rank, world, EP_TOKENS, range(n_layers))
                ms_n, _, _, _ = time_job(job_n, a.steps, warmup, barrier_max, min_ms=20.0)
                variants[name] = {"ms_per_step": ms_n, "value": EP_TOKENS * n_layers / (ms_n * 1e-3), "unit": UNIT}
                job_n.release()
            e2 = ep.q4_cuda_ep_error()
            if e2:
                raise SystemExit("expert-parallel error word %#x" % e2)
        else:
            variants["unavailable"] = "the ranks' buffers could not be mapped through CUDA IPC"
        ep.q4_cuda_ep_allreduce_mode(2)
        ep.q4_cuda_ep_split_routing(0)
        details["variants"] = variants
    if ep is not None:
        # the two-exchange form of the same job (tokens split over the ranks), for comparison
        job2 = BatchJob(pkg, model, ep, rank, world, EP_TOKENS, range(n_layers), form="a2a")
        ms2, _, launches2, _ = time_job(job2, a.steps, warmup, barrier_max, min_ms=20.0)
        details["two_exchange_form"] = {"ms_per_step": ms2, "value": EP_TOKENS * n_layers / (ms2 * 1e-3),
                                        "unit": UNIT, "launches_per_step": launches2}
        job2.release()
    if world > 1 and rank == 0 and not a.no_cpu:
        job.release()
        model.release()
        m1 = Model(dev, n_layers, 0)
        solo = BatchJob(pkg, m1, None, 0, 1, EP_TOKENS, range(n_layers))
        s_ms, s_e2e, _, _ = time_job(solo, a.steps, warmup, lambda v: v)

        def rel(got, want):
            return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))
        solo.enqueue(layers=[0])
        dev.sync()
        rel_l0 = rel(y_ep_l0, solo.output()[:job.rows])
        solo.step()
        dev.sync()
        rel_all = rel(y_ep, solo.output()[:job.rows])
        units1 = EP_TOKENS * n_layers
        details["one_gpu_same_job"] = {"value": units1 / (s_ms * 1e-3), "e2e": units1 / (s_e2e * 1e-3),
                                       "unit": UNIT, "ms_per_step": s_ms}
        details["speedup_vs_one_gpu"] = s_ms / ms
        # One layer from the same input rows: the two runs differ in the order of one fp32 sum per
        # output value.  This bound fails the run.  After a stack of layers the difference is
        # reported only: every layer's 8-bit quantiser turns a last-bit difference of its input
        # into a rounding flip now and then.
        details["parity_vs_one_gpu_rel_l2"] = rel_l0
        details["parity_vs_one_gpu_rel_l2_after_%d_layers" % n_layers] = rel_all
        if not rel_l0 <= 1e-5:
            raise SystemExit("expert-parallel result differs from the one-GPU result: rel-L2 %g" % rel_l0)
    barrier_max(0.0)
    if rank == 0:
        units = EP_TOKENS * n_layers
        print(json.dumps({
            "metric": METRIC, "value": units / (ms * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": a.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
            "config": config4(world, n_layers), "details": details, "clocks": clocks,
            "e2e": {"value": units / (ms_e2e * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": job.nb, "d2h_bytes_per_step": job.nb},
            "gpu_launches": int(launches * a.steps * repeats),
            "roofline": ep_roofline(world, n_layers, ms * 1e-3), "cpu_baseline": None}))
        sys.stdout.flush()
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
        try:
            atexit._run_exitfuncs()     # whatever the interpreter or its host registered for exit
        finally:
            os._exit(0)


# ------------------------------------------------------------------ the reference arm and main

def run_reference(a, pkg, rank, world, warmup):
    """The reference's own CPU implementation of the path on this host's cores (oracle/_ref: its
    q4_cpuexp.c / q4_quant.c compiled unmodified), on the configuration the GPU arm runs at this
    N: config 1 at N = 1, config 4 (64 tokens through the layers, window jobs) at N >= 2.  Each
    step is a bounded sample of the workload.  Rank 0 alone runs it."""
    if rank != 0:
        return
    steps = min(a.steps, 200)
    if world == 1:
        config, n_tok, jobs, scaling = CONFIG1, 1, 64, "weak"
        what = "%d layer-tokens per step (one-token jobs) over 2 layers of weights" % jobs
    else:
        config, n_tok, jobs, scaling = config4(world, a.layers or N_LAYERS), EP_TOKENS, 4, "strong"
        what = "%d layers of the step's %d per step, all 64 tokens, over 2 layers of weights" % (
            jobs, a.layers or N_LAYERS)
    # in a child with a time limit (the pool is the reference's own code and has been seen not to return)
    d = cpu_child("arm", 0.25 * steps, None, None, n_tok,
                  extra=["--cpu-jobs", str(jobs), "--cpu-steps", str(steps), "--cpu-warm", str(min(warmup, 3))])
    if "unavailable" in d:
        print(json.dumps({"impl": "reference", "unavailable": d["unavailable"]}))
        return
    t, t_router = d["t"], d["t_router"]
    lt = steps * jobs * n_tok
    val = lt / t
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": a.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": 1e3 * t / steps, "higher_is_better": True, "scaling": scaling,
        "vs_baseline": None, "dtype": DTYPE, "data": "synthetic", "config": config,
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": d["cores"], "kind": "reference",
                         "cpu_model": d["cpu_model"], "sample": "%d steps x %s" % (steps, what),
                         "router_ms": 1e3 * t_router / lt, "experts_ms": 1e3 * (t - t_router) / lt,
                         "omp_threads": d["omp_threads"]},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def dist_setup():
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")),
            int(os.environ.get("LOCAL_RANK", "0")))


def run_config1(a, pkg, local, warmup):
    dev = pkg.Device()
    lib = dev.lib
    model = Model(dev, a.layers)
    d1 = Decode1(pkg, model)
    k = a.steps
    sampler = ClockSampler(local)
    sampler.start()
    # --- device-resident: K consecutive layer-steps per set, sets repeated to >= 50 ms ---
    ms, repeats, timed_ms, launches = median_step(lib, lambda r: d1.enqueue_steps(k, r), k,
                                                  max(1, (warmup + k - 1) // k))
    # --- end to end through the one-layer host-buffer call, every step ---
    ke = min(k, 256)
    ms_e2e, rep_e2e = median_wall(lambda r: d1.e2e_steps(ke, r), ke, max(1, (min(warmup, 50) + ke - 1) // ke))
    ms_e2e_stack, _ = median_wall(d1.e2e_stack, model.n_layers, 2)
    # --- end to end through a session: the same kernel resident, a doorbell ring per step ---
    d1.session_begin()
    ms_e2e_ses, rep_e2e_ses = median_wall(lambda r: d1.session_steps(ke, r), ke,
                                          max(1, (min(warmup, 50) + ke - 1) // ke))
    d1.session_end()
    clocks = sampler.stop()
    err = lib.q4_cuda_device_error()
    if err:
        raise SystemExit("device error word %#x" % err)
    hbm, _, peak_src = read_peaks()
    achieved = STEP_BYTES / (ms * 1e-3) / 1e9
    tr = read_traffic("decode_stack_kernel.json")
    cpu_layers, cpu, details = None, None, {}
    if not a.no_cpu:
        cpu_layers = dump_layers(model.host_layers(range(min(2, model.n_layers))))
        cpu = cpu_child("layers", a.cpu_seconds, cpu_layers, d1.x_host, 1)
        if "unavailable" not in cpu:
            cpu["jobs_router_on_a_passive_openmp_team"] = cpu_probe_passive_omp(min(a.cpu_seconds, 5.0))
    details["repeats"] = repeats
    details["timed_ms"] = timed_ms
    details["steps_per_launch"] = min(k, model.n_layers)
    details["e2e_repeats"] = rep_e2e_ses
    details["e2e_api"] = ("q4_cuda_decode_session_step: the stack kernel stays resident, each step's 8 KB row goes "
                          "from host memory into the kernel and its 8 KB result back, one layer per step")
    details["e2e_one_launch_per_step"] = {"value": 1e3 / ms_e2e, "unit": UNIT, "repeats": rep_e2e,
                                          "what": "q4_cuda_decode_plan_host: one kernel launch per layer-step, "
                                                  "8 KB in and 8 KB out per call"}
    details["e2e_stack"] = {"value": 1e3 / ms_e2e_stack, "unit": UNIT,
                            "what": "one host-buffer call per token through all %d layers (8 KB in, 8 KB out per "
                                    "call)" % model.n_layers}
    d1.release()
    if not a.no_others:
        cs = 0.0 if a.no_cpu else min(a.cpu_seconds, 4.0)
        others = [measure_config0(pkg, model, cpu_layers, cs),
                  measure_batch(pkg, model, "verify", 5, 3, cpu_layers, cs),
                  measure_batch(pkg, model, "ep1", 3, 3, cpu_layers, cs)]
        model.release()
        m2 = Model(dev, 2)
        others.insert(2, measure_batch(pkg, m2, "prefill", 10, 3, None, cs))
        m2.release()
        details["other_workloads"] = others
    line = {
        "metric": METRIC, "value": 1e3 / ms, "unit": UNIT, "n_gpus": 1, "steps": k, "warmup": warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic", "config": dict(CONFIG1, layers_rotated=a.layers),
        "details": details, "clocks": clocks,
        "e2e": {"value": 1e3 / ms_e2e_ses, "unit": UNIT, "h2d_bytes_per_step": N_EMBD * 4,
                "d2h_bytes_per_step": N_EMBD * 4},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                     "traffic": tr.get("dram_bytes_per_layer_token") if tr else None,
                     "traffic_source": tr.get("source") if tr else None, "peak_source": peak_src,
                     "kernel": "moe_decode_stack_k, one launch per %d steps" % min(k, model.n_layers)},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=480)
    ap.add_argument("--warmup", type=int, default=48)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=N_LAYERS)
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU legs (and the one-GPU rerun at N >= 2)")
    ap.add_argument("--no-others", action="store_true", help="config 1 only: skip details.other_workloads")
    ap.add_argument("--workload", default="auto", choices=["auto", "config0", "verify", "prefill", "ep"],
                    help="one of the other configurations alone on one GPU (its entry is printed)")
    ap.add_argument("--cpu-probe", action="store_true", help=argparse.SUPPRESS)       # the child of a CPU leg
    ap.add_argument("--cpu-kind", default="layers", help=argparse.SUPPRESS)
    ap.add_argument("--cpu-dir", default="", help=argparse.SUPPRESS)
    ap.add_argument("--cpu-tokens", type=int, default=1, help=argparse.SUPPRESS)
    ap.add_argument("--cpu-nochain", action="store_true", help=argparse.SUPPRESS)
    ap.add_argument("--cpu-jobs", type=int, default=64, help=argparse.SUPPRESS)
    ap.add_argument("--cpu-steps", type=int, default=20, help=argparse.SUPPRESS)
    ap.add_argument("--cpu-warm", type=int, default=3, help=argparse.SUPPRESS)
    ap.add_argument("--watchdog-s", type=int, default=900,
                    help="dump every thread's stack to stderr and exit if the run takes longer than this")
    a = ap.parse_args()
    # A run that does not end is worse than one that fails: after 15 minutes say where every thread is
    # (stderr) and leave.  The default run takes about a minute.
    faulthandler.dump_traceback_later(a.watchdog_s, exit=True)
    rank, world, local = dist_setup()
    warmup = max(a.warmup, 3)
    if world > 1:       # one process per GPU: each sees only its own device
        os.environ["CUDA_VISIBLE_DEVICES"] = str(local)
    if a.cpu_probe:
        entry.build()
        cpu_probe_main(a)
        return
    entry.build()
    pkg = entry.load_package()
    if a.impl == "reference":
        run_reference(a, pkg, rank, world, warmup)
        return
    if world > 1:
        run_ep(a, pkg, rank, world, local, warmup)
        return
    if a.workload != "auto":
        dev = pkg.Device()
        cs = 0.0 if a.no_cpu else min(a.cpu_seconds, 4.0)
        if a.workload == "prefill":
            model = Model(dev, 2)
            out = measure_batch(pkg, model, "prefill", min(a.steps, 20), warmup, None, cs)
        else:
            model = Model(dev, a.layers)
            cl = dump_layers(model.host_layers(range(min(2, a.layers)))) if cs else None
            if a.workload == "config0":
                out = measure_config0(pkg, model, cl, cs)
            else:
                out = measure_batch(pkg, model, "verify" if a.workload == "verify" else "ep1", min(a.steps, 20),
                                    warmup, cl, cs)
        print(json.dumps(out))
        return
    run_config1(a, pkg, local, warmup)


if __name__ == "__main__":
    main()
