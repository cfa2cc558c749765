"""ctypes/numpy front-end of the CPU restatement of infr-cpu (``infr_cpu_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, the smoke check and the benchmark's
CPU-baseline leg.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libinfr_cpu_oracle.so")

F32, Q4K, Q6K, Q2_0 = 0, 12, 14, 27
BLOCK = {F32: (1, 4), Q4K: (256, 144), Q6K: (256, 210), Q2_0: (64, 18)}

_u8p = C.POINTER(C.c_uint8)
_i8p = C.POINTER(C.c_int8)
_u16p = C.POINTER(C.c_uint16)
_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)


def build(force: bool = False) -> str:
    """Compile the restatement with the committed Makefile (gcc, -ffp-contract=off)."""
    src = os.path.join(_HERE, "infr_cpu_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


def _p(a, t):
    return a.ctypes.data_as(t) if a is not None else None


class Oracle:
    def __init__(self):
        build()
        L = C.CDLL(_LIB_PATH)
        self.L = L
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_k4.argtypes = [C.c_int, _u8p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        L.orc_dequant.argtypes = [C.c_int, _u8p, C.c_size_t, _f32p]
        L.orc_quantize_q8.argtypes = [_f32p, C.c_size_t, _i8p, _f32p, _i32p, _i32p]
        L.orc_quantize_q8_32.argtypes = [_f32p, C.c_size_t, _i8p, _f32p, _i32p]
        L.orc_quantize_q8_1.argtypes = [_f32p, C.c_size_t, _i8p, _u16p, _u16p]
        L.orc_vec_dot_q4k.restype = C.c_float
        L.orc_vec_dot_q4k.argtypes = [_u8p, _i8p, _f32p, _i32p, C.c_size_t, _i32p, _i32p]
        L.orc_vec_dot_q6k.restype = C.c_float
        L.orc_vec_dot_q6k.argtypes = [_u8p, _i8p, _f32p, C.c_size_t, _i32p]
        L.orc_vec_dot_q2_0.restype = C.c_float
        L.orc_vec_dot_q2_0.argtypes = [_u8p, _i8p, _f32p, _i32p, C.c_size_t, _i32p]
        L.orc_dot.restype = C.c_float
        L.orc_dot.argtypes = [_f32p, _f32p, C.c_size_t]
        L.orc_gated_silu.restype = C.c_float
        L.orc_gated_silu.argtypes = [C.c_float, C.c_float]
        L.orc_ref_linear_f64.argtypes = [_f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t, _f32p]
        L.orc_linear.argtypes = [C.c_int, _u8p, _f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t,
                                 C.c_int, C.c_int]
        L.orc_mmq_q8_1.argtypes = [C.c_int, _u8p, _i8p, _u16p, _u16p, _f32p, C.c_size_t, C.c_size_t,
                                   C.c_size_t, _i32p]
        L.orc_moe_ffn.argtypes = [_f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                  C.c_size_t, C.c_int, _u8p, C.c_int, _u8p, C.c_int, _u8p, C.c_int,
                                  _u8p, C.c_float, C.c_int, C.c_int, _f32p, _i32p, _f32p, _f32p,
                                  C.c_int]
        L.orc_num_threads.restype = C.c_int
        L.orc_rms_norm.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, C.c_size_t, C.c_float]
        L.orc_rope.argtypes = [_f32p, _f32p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float, C.c_int]
        L.orc_write_kv_f16.argtypes = [_f32p, _u16p, C.c_size_t, C.c_size_t, C.c_size_t]
        L.orc_attention.argtypes = [_f32p, _u16p, _u16p, _f32p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                    C.c_float, C.c_size_t]
        L.orc_gated_act.argtypes = [_f32p, _f32p, _f32p, C.c_size_t]
        L.orc_add.argtypes = [_f32p, _f32p, _f32p, C.c_size_t]
        L.orc_argmax.argtypes = [_f32p, C.POINTER(C.c_uint32), C.c_size_t, C.c_size_t]

    # ---- scalars ---------------------------------------------------------------------------
    def f16_to_f32(self, h: int) -> float:
        return float(self.L.orc_f16_to_f32(h))

    def f32_to_f16(self, f: float) -> int:
        return int(self.L.orc_f32_to_f16(f))

    def k4(self, j: int, scales: np.ndarray):
        sc, m = C.c_uint32(), C.c_uint32()
        s = np.ascontiguousarray(scales, dtype=np.uint8)
        self.L.orc_k4(j, _p(s, _u8p), C.byref(sc), C.byref(m))
        return sc.value, m.value

    def num_threads(self) -> int:
        return int(self.L.orc_num_threads())

    # ---- formats ---------------------------------------------------------------------------
    def dequant(self, dt: int, raw: np.ndarray) -> np.ndarray:
        raw = np.ascontiguousarray(raw, dtype=np.uint8).ravel()
        be, bb = BLOCK[dt]
        nblk = raw.size // bb
        out = np.empty(nblk * be, dtype=np.float32)
        rc = self.L.orc_dequant(dt, _p(raw, _u8p), nblk, _p(out, _f32p))
        assert rc == 0
        return out

    def quantize_q8(self, x: np.ndarray):
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        n = x.size
        qs = np.empty(n, np.int8)
        d = np.empty(n // 256, np.float32)
        bs = np.empty(n // 32, np.int32)
        bs16 = np.empty(n // 16, np.int32)
        self.L.orc_quantize_q8(_p(x, _f32p), n, _p(qs, _i8p), _p(d, _f32p), _p(bs, _i32p), _p(bs16, _i32p))
        return qs, d, bs, bs16

    def quantize_q8_32(self, x: np.ndarray):
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        n = x.size
        qs = np.empty(n, np.int8)
        d = np.empty(n // 32, np.float32)
        bs = np.empty(n // 32, np.int32)
        self.L.orc_quantize_q8_32(_p(x, _f32p), n, _p(qs, _i8p), _p(d, _f32p), _p(bs, _i32p))
        return qs, d, bs

    def quantize_q8_1(self, x: np.ndarray):
        x = np.ascontiguousarray(x, dtype=np.float32).ravel()
        n = x.size
        qs = np.empty(n, np.int8)
        d = np.empty(n // 32, np.uint16)
        s = np.empty(n // 32, np.uint16)
        self.L.orc_quantize_q8_1(_p(x, _f32p), n, _p(qs, _i8p), _p(d, _u16p), _p(s, _u16p))
        return qs, d, s

    # ---- dots ------------------------------------------------------------------------------
    def vec_dot_q4k(self, row, q8, in_f, want_acc=False):
        row = np.ascontiguousarray(row, np.uint8)
        qs, d, bs = q8[0], q8[1], q8[2]
        sd = np.empty(in_f // 256, np.int32) if want_acc else None
        sm = np.empty(in_f // 256, np.int32) if want_acc else None
        v = self.L.orc_vec_dot_q4k(_p(row, _u8p), _p(qs, _i8p), _p(d, _f32p), _p(bs, _i32p), in_f,
                                   _p(sd, _i32p), _p(sm, _i32p))
        return (np.float32(v), sd, sm) if want_acc else np.float32(v)

    def vec_dot_q6k(self, row, q8, in_f, want_acc=False):
        row = np.ascontiguousarray(row, np.uint8)
        qs, d = q8[0], q8[1]
        acc = np.empty(in_f // 256, np.int32) if want_acc else None
        v = self.L.orc_vec_dot_q6k(_p(row, _u8p), _p(qs, _i8p), _p(d, _f32p), in_f, _p(acc, _i32p))
        return (np.float32(v), acc) if want_acc else np.float32(v)

    def vec_dot_q2_0(self, row, q8x32, in_f, want_acc=False):
        row = np.ascontiguousarray(row, np.uint8)
        qs, d, bs = q8x32
        acc = np.empty(in_f // 32, np.int32) if want_acc else None
        v = self.L.orc_vec_dot_q2_0(_p(row, _u8p), _p(qs, _i8p), _p(d, _f32p), _p(bs, _i32p), in_f,
                                    _p(acc, _i32p))
        return (np.float32(v), acc) if want_acc else np.float32(v)

    def dot(self, a, b) -> np.float32:
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        return np.float32(self.L.orc_dot(_p(a, _f32p), _p(b, _f32p), a.size))

    def gated_silu(self, g: float, u: float) -> np.float32:
        return np.float32(self.L.orc_gated_silu(g, u))

    # ---- Op::Linear ------------------------------------------------------------------------
    def linear(self, dt, w, x, m, in_f, out_f, reference=False, threads=0) -> np.ndarray:
        w = np.ascontiguousarray(w, np.uint8).ravel()
        x = np.ascontiguousarray(x, np.float32).ravel()
        out = np.empty((m, out_f), np.float32)
        rc = self.L.orc_linear(dt, _p(w, _u8p), _p(x, _f32p), _p(out, _f32p), m, in_f, out_f,
                               1 if reference else 0, threads)
        assert rc == 0, rc
        return out

    def ref_linear_f64(self, x, w, m, in_f, out_f) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32).ravel()
        w = np.ascontiguousarray(w, np.float32).ravel()
        out = np.empty((m, out_f), np.float32)
        self.L.orc_ref_linear_f64(_p(x, _f32p), _p(w, _f32p), m, in_f, out_f, _p(out, _f32p))
        return out

    def mmq_q8_1(self, dt, w, qa, dact, sact, m, in_f, out_f, want_qsum=False):
        w = np.ascontiguousarray(w, np.uint8).ravel()
        out = np.empty((m, out_f), np.float32)
        per = in_f // (16 if dt == Q6K else 32)
        qsum = np.empty((m, out_f, per), np.int32) if want_qsum else None
        rc = self.L.orc_mmq_q8_1(dt, _p(w, _u8p), _p(qa, _i8p), _p(dact, _u16p), _p(sact, _u16p),
                                 _p(out, _f32p), m, in_f, out_f, _p(qsum, _i32p))
        assert rc == 0
        return (out, qsum) if want_qsum else out

    # ---- Op::MoeFfn ------------------------------------------------------------------------
    def moe_ffn(self, x, router, gate, up, down, *, rows, ne, n_expert, n_used, n_ff_exp, wdt=Q4K, down_dt=None,
                scale=1.0, norm_w=True, reference=False, router_x=None, threads=0):
        x = np.ascontiguousarray(x, np.float32).ravel()
        rx = x if router_x is None else np.ascontiguousarray(router_x, np.float32).ravel()
        router = np.ascontiguousarray(router, np.float32).ravel().view(np.uint8)
        gate = np.ascontiguousarray(gate, np.uint8).ravel()
        up = np.ascontiguousarray(up, np.uint8).ravel()
        down = np.ascontiguousarray(down, np.uint8).ravel()
        dst = np.empty((rows, ne), np.float32)
        ids = np.empty((rows, n_used), np.int32)
        wts = np.empty((rows, n_used), np.float32)
        logits = np.empty((rows, n_expert), np.float32)
        rc = self.L.orc_moe_ffn(_p(x, _f32p), _p(rx, _f32p), rows, ne, n_expert, n_used, n_ff_exp, F32,
                                _p(router, _u8p), wdt, _p(gate, _u8p), wdt, _p(up, _u8p), wdt if down_dt is None else down_dt,
                                _p(down, _u8p), scale, int(norm_w), int(reference), _p(dst, _f32p),
                                _p(ids, _i32p), _p(wts, _f32p), _p(logits, _f32p), threads)
        assert rc == 0
        return dst, ids, wts, logits

    # ---- dense decode-step ops -------------------------------------------------------------
    def rms_norm(self, x, w, eps) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        w = np.ascontiguousarray(w, np.float32)
        rows, dim = x.reshape(-1, w.size).shape
        out = np.empty_like(x)
        self.L.orc_rms_norm(_p(x, _f32p), _p(w, _f32p), _p(out, _f32p), rows, dim, eps)
        return out

    def rope(self, x, pos, n_head, head_dim, rope_dim, theta, neox=False) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        pos = np.ascontiguousarray(pos, np.float32)
        out = np.empty_like(x)
        self.L.orc_rope(_p(x, _f32p), _p(pos, _f32p), _p(out, _f32p), pos.size, n_head, head_dim, rope_dim, theta,
                        int(neox))
        return out

    def write_kv_f16(self, src, cache, rows, row_stride, pos):
        """Writes into `cache` (uint16 array, modified in place)."""
        src = np.ascontiguousarray(src, np.float32)
        assert cache.dtype == np.uint16 and cache.flags.c_contiguous
        self.L.orc_write_kv_f16(_p(src, _f32p), _p(cache, _u16p), rows, row_stride, pos)

    def attention(self, q, k_cache, v_cache, rows, n_head, n_kv, head_dim, scale, pos) -> np.ndarray:
        q = np.ascontiguousarray(q, np.float32)
        assert k_cache.dtype == np.uint16 and v_cache.dtype == np.uint16
        out = np.empty((rows, n_head * head_dim), np.float32)
        self.L.orc_attention(_p(q, _f32p), _p(k_cache, _u16p), _p(v_cache, _u16p), _p(out, _f32p), rows, n_head, n_kv,
                             head_dim, scale, pos)
        return out

    def gated_act(self, gate, up) -> np.ndarray:
        gate = np.ascontiguousarray(gate, np.float32)
        up = np.ascontiguousarray(up, np.float32)
        out = np.empty_like(gate)
        self.L.orc_gated_act(_p(gate, _f32p), _p(up, _f32p), _p(out, _f32p), gate.size)
        return out

    def add(self, a, b) -> np.ndarray:
        a = np.ascontiguousarray(a, np.float32)
        b = np.ascontiguousarray(b, np.float32)
        out = np.empty_like(a)
        self.L.orc_add(_p(a, _f32p), _p(b, _f32p), _p(out, _f32p), a.size)
        return out

    def argmax(self, x, n) -> np.ndarray:
        x = np.ascontiguousarray(x, np.float32)
        rows = x.size // n
        out = np.empty(rows, np.uint32)
        self.L.orc_argmax(_p(x, _f32p), out.ctypes.data_as(C.POINTER(C.c_uint32)), n, rows)
        return out
