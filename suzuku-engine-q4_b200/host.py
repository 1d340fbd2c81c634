"""Host side of the MoE path above the C ABI, in the shape of the reference
engine's all-GPU layer routine (src/q4_moe.c:2052-2133, q4_moe_layer_dev with
CPU experts off): experts live in a fixed-stride device arena, slot e holds
routed expert e and one extra slot holds the shared expert; a layer call is
RMSNorm -> router -> top-k -> routed + shared experts.

Everything that computes goes through libq4cuda.so; numpy only carries bytes to
and from the device.
"""
import ctypes as C

import numpy as np

from . import capi, synth

IQ3_S = 21
F32 = 0


class Device:
    """Thin owner of the library handle plus upload/download helpers."""

    def __init__(self):
        self.lib = capi.load()
        if not self.lib.q4_hip_init():
            raise RuntimeError("q4_hip_init failed: a CUDA sm_100 device is required "
                               "(this library has no CPU path)")
        self._live = []

    def malloc(self, nbytes):
        p = self.lib.q4_hip_malloc(nbytes)
        if not p:
            raise MemoryError("q4_hip_malloc(%d)" % nbytes)
        self._live.append(p)
        return p

    def free(self, p):
        self.lib.q4_hip_free(p)
        self._live.remove(p)

    def upload(self, arr):
        arr = np.ascontiguousarray(arr)
        p = self.malloc(max(arr.nbytes, 4))
        if arr.nbytes and not self.lib.q4_hip_h2d(p, arr.ctypes.data, arr.nbytes):
            raise RuntimeError("q4_hip_h2d")
        return p

    def write(self, p, arr):
        arr = np.ascontiguousarray(arr)
        if not self.lib.q4_hip_h2d(p, arr.ctypes.data, arr.nbytes):
            raise RuntimeError("q4_hip_h2d")

    def download(self, p, shape, dtype):
        out = np.empty(shape, dtype)
        if out.nbytes and not self.lib.q4_hip_d2h(out.ctypes.data, p, out.nbytes):
            raise RuntimeError("q4_hip_d2h")
        return out

    def sync(self):
        self.lib.q4_hip_sync()

    def release(self):
        for p in list(self._live):
            self.lib.q4_hip_free(p)
        self._live = []


class MoeLayer:
    """One MoE layer resident on the device.

    experts: uint8 [n_expert, pack_bytes]; shared: uint8 [pack_bytes] or None;
    router: fp32 [n_expert, n_embd]; norm_w: fp32 [n_embd] or None.
    arena: which library arena (0..3) holds this layer's packs.
    """

    def __init__(self, dev, experts, shared, router, norm_w, n_embd, n_ff, topk, eps=1e-6,
                 arena=0):
        self.dev = dev
        lib = dev.lib
        self.n_expert = int(experts.shape[0])
        self.n_embd, self.n_ff, self.topk, self.eps = n_embd, n_ff, topk, eps
        self.pack = synth.expert_pack_bytes(n_embd, n_ff)
        assert experts.shape[1] == self.pack
        self.arena = arena
        n_slots = self.n_expert + (1 if shared is not None else 0)
        if not lib.q4_hip_experts_alloc_a(arena, n_slots, self.pack):
            raise MemoryError("q4_hip_experts_alloc_a")
        for e in range(self.n_expert):
            row = np.ascontiguousarray(experts[e])
            if not lib.q4_hip_experts_put_a(arena, e, row.ctypes.data, self.pack):
                raise RuntimeError("q4_hip_experts_put_a")
        self.shared_slot = -1
        if shared is not None:
            self.shared_slot = self.n_expert
            sh = np.ascontiguousarray(shared)
            if not lib.q4_hip_experts_put_a(arena, self.shared_slot, sh.ctypes.data, self.pack):
                raise RuntimeError("q4_hip_experts_put_a")
        self.base = lib.q4_hip_experts_base_a(arena)
        self.stride = lib.q4_hip_experts_stride_a(arena)
        rb = synth.iq3s_row_bytes(n_embd)
        self.og, self.ou, self.od = 0, n_ff * rb, 2 * n_ff * rb
        self.d_router = dev.upload(router.astype(np.float32))
        self.d_norm = dev.upload(norm_w.astype(np.float32)) if norm_w is not None else None
        self.d_x = dev.malloc(4 * n_embd)
        self.d_y = dev.malloc(4 * n_embd)
        self.d_h = dev.malloc(4 * 64 * n_ff)
        self.d_ids = dev.malloc(4 * 64)
        self.d_wts = dev.malloc(4 * 64)

    def close(self):
        self.dev.lib.q4_hip_experts_free_a(self.arena)

    # --- the engine's fine-grained call (src/q4.h:930-935) ---
    def exec_experts(self, x, slots, wts):
        """y = sum_e wts[e] * FFN_slot[e](x), host-side expert list."""
        lib, dev = self.dev.lib, self.dev
        dev.write(self.d_x, np.asarray(x, np.float32))
        if not lib.q4_hip_fill(self.d_y, 0.0, self.n_embd):
            raise RuntimeError("q4_hip_fill")
        slots = np.ascontiguousarray(slots, np.int32)
        wts = np.ascontiguousarray(wts, np.float32)
        ok = lib.q4_hip_moe_exec(self.base, self.stride, slots.ctypes.data, wts.ctypes.data,
                                 slots.size, IQ3_S, self.og, IQ3_S, self.ou, IQ3_S, self.od,
                                 self.d_x, self.d_h, None, None, self.d_y, self.n_ff,
                                 self.n_embd, self.n_embd)
        if not ok:
            raise RuntimeError("q4_hip_moe_exec refused")
        y = dev.download(self.d_y, (self.n_embd,), np.float32)
        h = dev.download(self.d_h, (slots.size, self.n_ff), np.float32)
        return y, h

    # --- the fused layer call ---
    def decode(self, x):
        """One token through norm -> router -> experts.  Returns (y, ids, wts)."""
        lib, dev = self.dev.lib, self.dev
        dev.write(self.d_x, np.asarray(x, np.float32))
        ok = lib.q4_cuda_moe_decode(self.base, self.stride, self.og, self.ou, self.od,
                                    self.shared_slot, self.d_x, self.d_norm, self.eps,
                                    self.d_router, self.n_expert, self.topk, self.n_embd,
                                    self.n_ff, self.d_y, self.d_ids, self.d_wts)
        if not ok:
            raise RuntimeError("q4_cuda_moe_decode refused")
        y = dev.download(self.d_y, (self.n_embd,), np.float32)
        ids = dev.download(self.d_ids, (self.topk,), np.int32)
        wts = dev.download(self.d_wts, (self.topk,), np.float32)
        return y, ids, wts


# ---- expert parallelism: the host-side statement of the partition (libq4cuda_ep.so
# implements the same rules on the device, csrc/q4b_ep.cu) ----
def ep_expert_range(rank, world, n_expert):
    """Experts [first, first + count) live on `rank`."""
    assert n_expert % world == 0
    count = n_expert // world
    return rank * count, count


def ep_local_picks(ids, wts, rank, world, n_expert, t_local, has_shared=True):
    """Picks of all tokens as seen by one rank.

    ids/wts: [T, topk] for all T = world * t_local tokens (token t is owned by rank
    t // t_local).  Returns (lids, lw) of shape [T, topk + 1]: the local slot of each
    pick that lives on this rank (else -1, weight 0), and in the last column the shared
    expert (local slot count, weight 1) for the tokens this rank owns."""
    first, count = ep_expert_range(rank, world, n_expert)
    T, topk = ids.shape
    lids = np.full((T, topk + 1), -1, np.int32)
    lw = np.zeros((T, topk + 1), np.float32)
    mine = (ids >= first) & (ids < first + count)
    lids[:, :topk][mine] = (ids - first)[mine]
    lw[:, :topk][mine] = wts[mine]
    if has_shared:
        own = np.arange(T) // t_local == rank
        lids[own, topk] = count
        lw[own, topk] = 1.0
    return lids, lw
