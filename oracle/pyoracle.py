"""ctypes front end for the CPU checkers (test infrastructure only).

`Oracle` wraps oracle/_build/libq4oracle.so, the plain-C restatement.
`Reference` wraps oracle/_ref/libq4ref.so, the reference engine's own CPU expert
path compiled from its sources; `reference()` returns None when that library was
never built (no reference checkout on this machine and no prebuilt copy).

Only tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
import ctypes as C
import os

import numpy as np

from . import build as _build

Q8_DTYPE = np.dtype([("q", np.int8, (32,)), ("d", np.float32), ("bs", np.int32)])
assert Q8_DTYPE.itemsize == 40

_u8p = C.POINTER(C.c_uint8)
_f32p = C.POINTER(C.c_float)
_i32p = C.POINTER(C.c_int32)
_u32p = C.POINTER(C.c_uint32)
_i8p = C.POINTER(C.c_int8)


def _p(a, t):
    return a.ctypes.data_as(t)


def _u8(a):
    a = np.ascontiguousarray(a, dtype=np.uint8)
    return a


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class Oracle:
    def __init__(self):
        self.lib = C.CDLL(_build.build_oracle())
        L = self.lib
        L.q4o_iq3s_grid.restype = C.c_uint32
        L.q4o_iq3s_grid.argtypes = [C.c_uint32]
        L.q4o_f16_to_f32.restype = C.c_float
        L.q4o_f16_to_f32.argtypes = [C.c_uint16]
        L.q4o_iq3s_dot8.restype = C.c_float
        L.q4o_iq3s_dot8.argtypes = [_u8p, C.c_void_p, C.c_uint64]
        L.q4o_iq3s_dot_mmq.restype = C.c_float
        L.q4o_iq3s_dot_mmq.argtypes = [_u8p, _i8p, _f32p, C.c_uint64]
        L.q4o_silu.restype = C.c_float
        L.q4o_silu.argtypes = [C.c_float]
        L.q4o_iq4nl_dot8.restype = C.c_float
        L.q4o_iq4nl_dot8.argtypes = [_u8p, C.c_void_p, C.c_uint64]
        L.q4o_dot8_t.restype = C.c_float
        L.q4o_dot8_t.argtypes = [C.c_uint32, _u8p, C.c_void_p, C.c_uint64]
        L.q4o_mv_row.restype = C.c_float
        L.q4o_mv_row.argtypes = [C.c_uint32, _u8p, C.c_uint64, _i8p, _f32p, C.c_void_p]
        L.q4o_mv_geometry.restype = C.c_int

    def grid(self):
        return np.array([self.lib.q4o_iq3s_grid(i) for i in range(512)], dtype=np.uint32)

    def f16_to_f32(self, h):
        return self.lib.q4o_f16_to_f32(int(h))

    def unpack(self, blk):
        blk = _u8(blk)
        w = np.zeros(256, np.int8)
        ls = np.zeros(8, np.uint8)
        d = C.c_float()
        self.lib.q4o_iq3s_unpack(_p(blk, _u8p), _p(w, _i8p), _p(ls, _u8p), C.byref(d))
        return w, ls, d.value

    def dequant_row(self, row, n):
        row = _u8(row)
        out = np.zeros(n, np.float32)
        self.lib.q4o_iq3s_dequant_row(_p(row, _u8p), C.c_uint64(n), _p(out, _f32p))
        return out

    def quant8(self, x):
        x = _f32(x).ravel()
        out = np.zeros(x.size // 32, Q8_DTYPE)
        self.lib.q4o_quant8(_p(x, _f32p), C.c_uint64(x.size), C.c_void_p(out.ctypes.data))
        return out

    def group_idot(self, row, xq, n):
        row = _u8(row)
        out = np.zeros(n // 32, np.int32)
        self.lib.q4o_iq3s_group_idot(_p(row, _u8p), C.c_void_p(xq.ctypes.data),
                                     C.c_uint64(n), _p(out, _i32p))
        return out

    def dot8(self, row, xq, n):
        row = _u8(row)
        return float(self.lib.q4o_iq3s_dot8(_p(row, _u8p), C.c_void_p(xq.ctypes.data),
                                            C.c_uint64(n)))

    # ---- IQ4_NL (a routed expert's down projection may use it) ----
    def iq4nl_dequant_row(self, row, n):
        row = _u8(row)
        out = np.zeros(n, np.float32)
        self.lib.q4o_iq4nl_dequant_row(_p(row, _u8p), C.c_uint64(n), _p(out, _f32p))
        return out

    def iq4nl_group_idot(self, row, xq, n):
        row = _u8(row)
        out = np.zeros(n // 32, np.int32)
        self.lib.q4o_iq4nl_group_idot(_p(row, _u8p), C.c_void_p(xq.ctypes.data), C.c_uint64(n),
                                      _p(out, _i32p))
        return out

    def iq4nl_dot8(self, row, xq, n):
        row = _u8(row)
        return float(self.lib.q4o_iq4nl_dot8(_p(row, _u8p), C.c_void_p(xq.ctypes.data), C.c_uint64(n)))

    def expert_job_t(self, packs, wts, x, n_embd, n_ff, down_type, gu_type=21):
        packs = [_u8(p) for p in packs]
        arr = (C.c_void_p * len(packs))(*[p.ctypes.data for p in packs])
        wts = _f32(wts)
        x = _f32(x)
        y = np.zeros(n_embd, np.float32)
        self.lib.q4o_expert_job_t(arr, _p(wts, _f32p), C.c_uint32(len(packs)), _p(x, _f32p),
                                  C.c_uint32(n_embd), C.c_uint32(n_ff), C.c_uint32(gu_type),
                                  C.c_uint32(down_type), _p(y, _f32p))
        return y

    # ---- IQ4_XS ----
    def iq4xs_dequant_row(self, row, n):
        row = _u8(row)
        out = np.zeros(n, np.float32)
        self.lib.q4o_iq4xs_dequant_row(_p(row, _u8p), C.c_uint64(n), _p(out, _f32p))
        return out

    def iq4xs_group_idot(self, row, xq, n):
        row = _u8(row)
        out = np.zeros(n // 32, np.int32)
        self.lib.q4o_iq4xs_group_idot(_p(row, _u8p), C.c_void_p(xq.ctypes.data), C.c_uint64(n),
                                      _p(out, _i32p))
        return out

    def dot8_t(self, type_id, row, xq, n):
        row = _u8(row)
        return float(self.lib.q4o_dot8_t(C.c_uint32(type_id), _p(row, _u8p), C.c_void_p(xq.ctypes.data),
                                         C.c_uint64(n)))

    def matvec8(self, mat, rows, xq, n):
        """rows x n IQ3_S matrix times one quantised activation vector."""
        mat = _u8(mat)
        rb = n // 256 * 110
        out = np.zeros(rows, np.float32)
        base = mat.ctypes.data
        for r in range(rows):
            out[r] = self.lib.q4o_iq3s_dot8(C.cast(base + r * rb, _u8p),
                                            C.c_void_p(xq.ctypes.data), C.c_uint64(n))
        return out

    def expert_ffn(self, pack, xq, n_embd, n_ff, wt, y):
        pack = _u8(pack)
        h = np.zeros(n_ff, np.float32)
        hq = np.zeros(n_ff // 32, Q8_DTYPE)
        self.lib.q4o_expert_ffn(_p(pack, _u8p), C.c_void_p(xq.ctypes.data),
                                C.c_uint32(n_embd), C.c_uint32(n_ff), C.c_float(wt),
                                _p(y, _f32p), _p(h, _f32p), C.c_void_p(hq.ctypes.data))
        return h, hq

    def expert_job(self, packs, wts, x, n_embd, n_ff):
        packs = [_u8(p) for p in packs]
        arr = (C.c_void_p * len(packs))(*[p.ctypes.data for p in packs])
        wts = _f32(wts)
        x = _f32(x)
        y = np.zeros(n_embd, np.float32)
        self.lib.q4o_expert_job(arr, _p(wts, _f32p), C.c_uint32(len(packs)), _p(x, _f32p),
                                C.c_uint32(n_embd), C.c_uint32(n_ff), _p(y, _f32p))
        return y

    def rms_norm(self, x, w, eps):
        x = _f32(x)
        y = np.zeros_like(x)
        wp = _p(_f32(w), _f32p) if w is not None else None
        self.lib.q4o_rms_norm(_p(x, _f32p), wp, _p(y, _f32p), C.c_uint64(x.size), C.c_float(eps))
        return y

    def gemv_f32(self, W, x):
        W = _f32(W)
        x = _f32(x)
        y = np.zeros(W.shape[0], np.float32)
        self.lib.q4o_gemv_f32(_p(W, _f32p), C.c_uint64(W.shape[0]), C.c_uint64(W.shape[1]),
                              _p(x, _f32p), _p(y, _f32p))
        return y

    def softmax(self, x):
        x = _f32(x).copy()
        self.lib.q4o_softmax(_p(x, _f32p), C.c_uint64(x.size))
        return x

    def topk(self, p, k, renorm=True):
        p = _f32(p)
        ids = np.zeros(k, np.int32)
        wts = np.zeros(k, np.float32)
        self.lib.q4o_topk(_p(p, _f32p), C.c_uint32(p.size), C.c_uint32(k), _p(ids, _i32p),
                          _p(wts, _f32p), C.c_int(1 if renorm else 0))
        return ids, wts

    def moe_layer(self, x, norm_w, eps, router_w, topk, experts, shared, n_embd, n_ff):
        """experts: uint8 array [n_expert, pack_bytes]; shared: uint8 [pack_bytes] or None."""
        experts = _u8(experts)
        n_expert = experts.shape[0]
        x = _f32(x)
        norm_w = _f32(norm_w)
        router_w = _f32(router_w)
        y = np.zeros(n_embd, np.float32)
        ids = np.zeros(topk, np.int32)
        wts = np.zeros(topk, np.float32)
        xn = np.zeros(n_embd, np.float32)
        sh = _u8(shared) if shared is not None else None
        self.lib.q4o_moe_layer(_p(x, _f32p), _p(norm_w, _f32p), C.c_float(eps),
                               _p(router_w, _f32p), C.c_uint32(n_expert), C.c_uint32(topk),
                               _p(experts, _u8p), C.c_uint64(experts.shape[1]),
                               _p(sh, _u8p) if sh is not None else None,
                               C.c_uint32(n_embd), C.c_uint32(n_ff), _p(y, _f32p),
                               _p(ids, _i32p), _p(wts, _f32p), _p(xn, _f32p))
        return y, ids, wts, xn

    def quant8_mmq(self, x):
        x = _f32(x).ravel()
        q = np.zeros(x.size, np.int8)
        d = np.zeros(x.size // 32, np.float32)
        self.lib.q4o_quant8_mmq(_p(x, _f32p), C.c_uint64(x.size), _p(q, _i8p), _p(d, _f32p))
        return q, d

    # ---- dense product of up to 8 activation rows in 8-bit form (src/q4_mmvq.cu)
    def quant8_d(self, x):
        """(q int8 [n], d f32 [n/32], s16 i32 [n/16]) of one activation row."""
        x = _f32(x).ravel()
        q = np.zeros(x.size, np.int8)
        d = np.zeros(x.size // 32, np.float32)
        s16 = np.zeros(x.size // 16, np.int32)
        self.lib.q4o_quant8_d(_p(x, _f32p), C.c_uint64(x.size), _p(q, _i8p), _p(d, _f32p),
                              C.c_void_p(s16.ctypes.data))
        return q, d, s16

    def mv_geometry(self, type_id):
        bb, bv = C.c_uint32(), C.c_uint32()
        assert self.lib.q4o_mv_geometry(C.c_uint32(type_id), C.byref(bb), C.byref(bv))
        return bb.value, bv.value

    def mv_dequant_row(self, type_id, row, n):
        row = _u8(row)
        out = np.zeros(n, np.float32)
        self.lib.q4o_mv_dequant_row(C.c_uint32(type_id), _p(row, _u8p), C.c_uint64(n), _p(out, _f32p))
        return out

    def mv_rows(self, type_id, w, nrows, ncols, xs, scale=1.0):
        """y [n, nrows] = scale * W . q8(x[t]) in the order of src/q4_mmvq.cu:195-243."""
        w = _u8(w).reshape(nrows, -1)
        xs = _f32(xs).reshape(-1, ncols)
        y = np.zeros((xs.shape[0], nrows), np.float32)
        for t in range(xs.shape[0]):
            q, d, s16 = self.quant8_d(xs[t])
            for r in range(nrows):
                v = self.lib.q4o_mv_row(C.c_uint32(type_id), _p(w[r], _u8p), C.c_uint64(ncols), _p(q, _i8p),
                                        _p(d, _f32p), C.c_void_p(s16.ctypes.data))
                y[t, r] = np.float32(scale) * np.float32(v)
        return y

    # ---- IQ3_XXS (18), IQ2_S (22), Q2_0 (42)
    def dequant_row_x(self, type_id, row, n):
        row = _u8(row)
        out = np.zeros(n, np.float32)
        self.lib.q4o_dequant_row_x(C.c_uint32(type_id), _p(row, _u8p), C.c_uint64(n), _p(out, _f32p))
        return out

    def group_idot_x(self, type_id, row, xq, n):
        row = _u8(row)
        I = np.zeros(n // 32, np.int32)
        self.lib.q4o_group_idot_x(C.c_uint32(type_id), _p(row, _u8p), C.c_void_p(xq.ctypes.data), C.c_uint64(n),
                                  _p(I, _i32p))
        return I

    def dot_mmq(self, row, q, d, n):
        row = _u8(row)
        return float(self.lib.q4o_iq3s_dot_mmq(_p(row, _u8p), _p(q, _i8p), _p(d, _f32p),
                                               C.c_uint64(n)))


class Reference:
    """The reference's own CPU code.  Thread count of its worker pool is fixed at
    the first job of the process (environment variable Q4_CPU_THREADS)."""

    def __init__(self, path):
        self.lib = C.CDLL(path)
        L = self.lib
        assert L.q4ref_q8_bytes() == 40
        for name in ("q4ref_dot8", "q4ref_dot8_avx2"):
            f = getattr(L, name)
            f.restype = C.c_float
            f.argtypes = [_u8p, C.c_void_p, C.c_uint64]
        L.q4ref_dot_f32.restype = C.c_float
        L.q4ref_dot_f32.argtypes = [_u8p, _f32p, C.c_uint64]
        L.q4ref_dot8_t.restype = C.c_float
        L.q4ref_dot8_t.argtypes = [C.c_uint32, _u8p, C.c_void_p, C.c_uint64]
        L.q4ref_dot8_avx2_iq4nl.restype = C.c_float
        L.q4ref_dot8_avx2_iq4nl.argtypes = [_u8p, C.c_void_p, C.c_uint64]
        L.q4ref_dot8_avx2_iq4xs.restype = C.c_float
        L.q4ref_dot8_avx2_iq4xs.argtypes = [_u8p, C.c_void_p, C.c_uint64]
        L.q4ref_time_jobs.restype = C.c_double
        L.q4ref_time_layers.restype = C.c_double
        L.q4ref_time_layers_win.restype = C.c_double

    def quant8(self, x):
        x = _f32(x).ravel()
        out = np.zeros(x.size // 32, Q8_DTYPE)
        self.lib.q4ref_quant8(_p(x, _f32p), C.c_uint64(x.size), C.c_void_p(out.ctypes.data))
        return out

    def dot8(self, row, xq, n, avx2=False):
        row = _u8(row)
        f = self.lib.q4ref_dot8_avx2 if avx2 else self.lib.q4ref_dot8
        return float(f(_p(row, _u8p), C.c_void_p(xq.ctypes.data), C.c_uint64(n)))

    def set_down_type(self, type_id):
        """Type of the down projection of the packs handed to expert_job (21 IQ3_S, 20 IQ4_NL)."""
        self.lib.q4ref_set_down_type(C.c_uint32(type_id))

    def set_gu_type(self, type_id):
        """Type of the gate and up projections of the packs handed to expert_job."""
        self.lib.q4ref_set_gu_type(C.c_uint32(type_id))

    def dequant_row_t(self, type_id, row, n):
        row = _u8(row)
        out = np.zeros(n, np.float32)
        assert self.lib.q4ref_dequant_row_t(C.c_uint32(type_id), _p(row, _u8p), C.c_uint64(n), _p(out, _f32p))
        return out

    def dot8_t(self, type_id, row, xq, n, avx2_iq4nl=False, avx2_iq4xs=False):
        row = _u8(row)
        if avx2_iq4nl:
            return float(self.lib.q4ref_dot8_avx2_iq4nl(_p(row, _u8p), C.c_void_p(xq.ctypes.data), C.c_uint64(n)))
        if avx2_iq4xs:
            return float(self.lib.q4ref_dot8_avx2_iq4xs(_p(row, _u8p), C.c_void_p(xq.ctypes.data), C.c_uint64(n)))
        return float(self.lib.q4ref_dot8_t(C.c_uint32(type_id), _p(row, _u8p), C.c_void_p(xq.ctypes.data),
                                           C.c_uint64(n)))

    def dot_f32(self, row, x, n):
        row = _u8(row)
        x = _f32(x)
        return float(self.lib.q4ref_dot_f32(_p(row, _u8p), _p(x, _f32p), C.c_uint64(n)))

    def dequant_row(self, row, n):
        row = _u8(row)
        out = np.zeros(n, np.float32)
        ok = self.lib.q4ref_dequant_row(_p(row, _u8p), C.c_uint64(n), _p(out, _f32p))
        assert ok
        return out

    def gemv(self, type_id, w, nrows, ncols, x):
        w = np.ascontiguousarray(w)
        x = _f32(x)
        y = np.zeros(nrows, np.float32)
        ok = self.lib.q4ref_gemv(C.c_uint32(type_id), C.c_void_p(w.ctypes.data),
                                 C.c_uint64(nrows), C.c_uint64(ncols), _p(x, _f32p),
                                 _p(y, _f32p))
        assert ok
        return y

    def rms_norm(self, x, w, eps):
        x = _f32(x)
        y = np.zeros_like(x)
        self.lib.q4ref_rms_norm(_p(x, _f32p), _p(_f32(w), _f32p) if w is not None else None,
                                _p(y, _f32p), C.c_uint64(x.size), C.c_float(eps))
        return y

    def softmax(self, x):
        x = _f32(x).copy()
        self.lib.q4ref_softmax(_p(x, _f32p), C.c_uint64(x.size))
        return x

    def topk(self, p, k, renorm=True):
        p = _f32(p)
        ids = np.zeros(k, np.int32)
        wts = np.zeros(k, np.float32)
        self.lib.q4ref_topk(_p(p, _f32p), C.c_uint32(p.size), C.c_uint32(k), _p(ids, _i32p),
                            _p(wts, _f32p), C.c_int(1 if renorm else 0))
        return ids, wts

    def threads(self):
        return int(self.lib.q4ref_threads())

    def selftest(self):
        return int(self.lib.q4ref_selftest())

    @staticmethod
    def _table(packs):
        packs = [_u8(p) for p in packs]
        return packs, (C.c_void_p * len(packs))(*[p.ctypes.data for p in packs])

    def expert_job(self, packs, ids, wts, x, n_embd, n_ff):
        keep, arr = self._table(packs)
        ids = np.ascontiguousarray(ids, np.int32)
        wts = _f32(wts)
        x = _f32(x)
        y = np.zeros(n_embd, np.float32)
        rc = self.lib.q4ref_expert_job(arr, C.c_uint32(len(keep)), _p(ids, _i32p),
                                       _p(wts, _f32p), C.c_uint32(ids.size), _p(x, _f32p),
                                       C.c_uint32(n_embd), C.c_uint32(n_ff), _p(y, _f32p))
        assert rc == 0, rc
        return y

    def expert_job_win(self, packs, ids, wts, tn, x, n_embd, n_ff):
        keep, arr = self._table(packs)
        ids = np.ascontiguousarray(ids, np.int32)
        wts = _f32(wts)
        tn = np.ascontiguousarray(tn, np.uint32)
        x = _f32(x)
        y = np.zeros((tn.size, n_embd), np.float32)
        rc = self.lib.q4ref_expert_job_win(arr, C.c_uint32(len(keep)), _p(ids, _i32p),
                                           _p(wts, _f32p), _p(tn, _u32p), C.c_uint32(tn.size),
                                           _p(x, _f32p), C.c_uint32(n_embd), C.c_uint32(n_ff),
                                           _p(y, _f32p))
        assert rc == 0, rc
        return y

    def time_jobs(self, packs, ids, wts, k, x, n_embd, n_ff):
        """ids/wts: [jobs, k]; x: [n_x, n_embd].  Returns seconds for all jobs."""
        keep, arr = self._table(packs)
        ids = np.ascontiguousarray(ids, np.int32)
        wts = _f32(wts)
        x = _f32(x)
        y = np.zeros(n_embd, np.float32)
        t = self.lib.q4ref_time_jobs(arr, C.c_uint32(len(keep)), _p(ids, _i32p),
                                     _p(wts, _f32p), C.c_uint32(k), C.c_uint32(ids.shape[0]),
                                     _p(x, _f32p), C.c_uint32(x.shape[0]), C.c_uint32(n_embd),
                                     C.c_uint32(n_ff), _p(y, _f32p))
        assert t >= 0, t
        return float(t)


    def time_layers(self, layers, topk, jobs, x, n_embd, n_ff, eps=1e-6):
        """layers: list of dicts with 'experts' [E, pack], 'shared' [pack], 'router'
        [E, n_embd], 'norm_w' [n_embd].  Job j runs layer j % len(layers) on
        x[j % len(x)].  Returns (seconds, ids [jobs, topk], last y)."""
        n_expert = layers[0]["experts"].shape[0]
        keep = []
        ptrs = []
        for L in layers:
            ex = _u8(L["experts"])
            sh = _u8(L["shared"])
            keep += [ex, sh]
            ptrs += [ex.ctypes.data + e * ex.shape[1] for e in range(n_expert)]
            ptrs.append(sh.ctypes.data)
        arr = (C.c_void_p * len(ptrs))(*ptrs)
        routers = [_f32(L["router"]) for L in layers]
        norms = [_f32(L["norm_w"]) for L in layers]
        r_arr = (C.c_void_p * len(layers))(*[r.ctypes.data for r in routers])
        n_arr = (C.c_void_p * len(layers))(*[n.ctypes.data for n in norms])
        x = _f32(x)
        y = np.zeros(n_embd, np.float32)
        ids = np.zeros((jobs, topk), np.int32)
        t = self.lib.q4ref_time_layers(arr, C.c_uint32(len(layers)), C.c_uint32(n_expert), r_arr,
                                       n_arr, C.c_float(eps), C.c_uint32(topk), C.c_uint32(jobs),
                                       _p(x, _f32p), C.c_uint32(x.shape[0]), C.c_uint32(n_embd),
                                       C.c_uint32(n_ff), _p(y, _f32p), _p(ids, _i32p))
        assert t >= 0, t
        return float(t), ids, y

    def time_layers_win(self, layers, topk, steps, x, n_embd, n_ff, chain, eps=1e-6):
        """`steps` layer jobs of len(x) tokens each through the reference's host routing and its
        window jobs (q4_cpuex_dispatch_win).  Job j runs layer j % len(layers); chain: a job's
        output rows feed the next.  Returns (seconds, seconds spent in norm + router + top-k, y)."""
        n_expert = layers[0]["experts"].shape[0]
        keep, ptrs = [], []
        for L in layers:
            ex, sh = _u8(L["experts"]), _u8(L["shared"])
            keep += [ex, sh]
            ptrs += [ex.ctypes.data + e * ex.shape[1] for e in range(n_expert)]
            ptrs.append(sh.ctypes.data)
        arr = (C.c_void_p * len(ptrs))(*ptrs)
        routers = [_f32(L["router"]) for L in layers]
        norms = [_f32(L["norm_w"]) for L in layers]
        r_arr = (C.c_void_p * len(layers))(*[r.ctypes.data for r in routers])
        n_arr = (C.c_void_p * len(layers))(*[n.ctypes.data for n in norms])
        x = _f32(x)
        y = np.zeros_like(x)
        rs = C.c_double(0.0)
        t = self.lib.q4ref_time_layers_win(arr, C.c_uint32(len(layers)), C.c_uint32(n_expert), r_arr, n_arr,
                                           C.c_float(eps), C.c_uint32(topk), C.c_uint32(steps), _p(x, _f32p),
                                           C.c_uint32(x.shape[0]), C.c_uint32(n_embd), C.c_uint32(n_ff),
                                           C.c_int(1 if chain else 0), _p(y, _f32p), C.byref(rs))
        assert t >= 0, t
        return float(t), float(rs.value), y


_ORACLE = None
_REF = False


def oracle():
    global _ORACLE
    if _ORACLE is None:
        _ORACLE = Oracle()
    return _ORACLE


def reference():
    """The compiled reference CPU path, or None when unavailable."""
    global _REF
    if _REF is False:
        path = _build.build_ref()
        _REF = Reference(path) if path else None
    return _REF
