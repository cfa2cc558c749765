"""infr_b200 — sm_100a implementation of infr's GGUF block-quantized matmul path.

The product is ``libinfr_cuda.so`` (hand-written CUDA kernels behind a C ABI, ``include/infr_cuda.h``).
This package is the thin ctypes binding used by the tests and the benchmark; its class
:class:`CudaBackend` mirrors the reference's ``trait Backend``
(crates/infr-core/src/backend.rs:486-662): ``name / capabilities / alloc / upload / download /
compile / execute / sync`` with the same argument meaning and error behaviour (errors raise
:class:`BackendError`, the analogue of ``Err(Error::Backend(..))``; nothing falls back to the CPU).
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from . import synth  # noqa: F401
from .synth import F32, Q2_0, Q4K, Q6K

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libinfr_cuda.so")

ACT_INT8, ACT_F32 = 0, 1
TK_INPUT, TK_WEIGHT, TK_INTERNAL, TK_OUTPUT = 0, 1, 2, 3
USAGE_WEIGHTS, USAGE_ACTIVATIONS, USAGE_KV, USAGE_READBACK = 0, 1, 2, 3
OP_LINEAR, OP_MOE_FFN, OP_RMS_NORM, OP_ROPE, OP_WRITE_KV, OP_ATTENTION, OP_GATED_ACT, OP_ADD, OP_ARGMAX, OP_COPY = range(1, 11)
F16, I32 = 1, 3
E_INVALID, E_UNSUPPORTED, E_OOM, E_CUDA, E_NCCL, E_TIMEOUT = -1, -2, -3, -4, -5, -6

# Every symbol include/infr_cuda.h declares (checked by the CPU test-suite against the built library).
EXPORTED_SYMBOLS = [
    "infr_cuda_create", "infr_cuda_destroy", "infr_cuda_get_caps", "infr_cuda_last_error",
    "infr_cuda_alloc", "infr_cuda_alloc_uninit", "infr_cuda_free", "infr_cuda_buf_len",
    "infr_cuda_buf_device_ptr", "infr_cuda_wrap", "infr_cuda_stream", "infr_cuda_comm_create", "infr_cuda_comm_export", "infr_cuda_comm_connect", "infr_cuda_comm_connect_silent",
    "infr_cuda_all_reduce_f32", "infr_cuda_comm_destroy", "infr_cuda_upload", "infr_cuda_upload_at", "infr_cuda_download",
    "infr_cuda_copy", "infr_cuda_host_alloc", "infr_cuda_host_free", "infr_cuda_sync", "infr_cuda_compile", "infr_cuda_plan_free", "infr_cuda_execute",
    "infr_cuda_quantize_q8", "infr_cuda_quantize_q8_1", "infr_cuda_gemv", "infr_cuda_gemv_q8", "infr_cuda_gemv_q8_pair", "infr_cuda_gemv_noalloc", "infr_cuda_gemv_block_acc",
    "infr_cuda_linear", "infr_cuda_linear_pair", "infr_cuda_moe_ffn", "infr_cuda_capture_begin", "infr_cuda_capture_end", "infr_cuda_graph_launch",
    "infr_cuda_graph_free", "infr_cuda_timer_start", "infr_cuda_timer_stop", "infr_cuda_flush_l2",
    "infr_cuda_launch_count", "infr_cuda_tensor_peak_i8",
    "infr_cuda_rms_norm", "infr_cuda_add_rms_norm", "infr_cuda_rope", "infr_cuda_write_kv", "infr_cuda_attention", "infr_cuda_rope_write_kv",
    "infr_cuda_gated_act", "infr_cuda_add", "infr_cuda_argmax", "infr_cuda_add_rms_norm_q8", "infr_cuda_gemv_q8_push", "infr_cuda_add_rms_norm_q8_pull", "infr_cuda_gated_act_q8", "infr_cuda_attention_q8",
    "infr_cuda_attention_seqpos", "infr_cuda_attention_seqpos_q8", "infr_cuda_attention_paged", "infr_cuda_rope_write_kv_paged",
    "infr_gguf_open", "infr_gguf_close", "infr_gguf_version", "infr_gguf_alignment", "infr_gguf_tensor_count", "infr_gguf_tensor_at", "infr_gguf_find",
    "infr_gguf_tensor_data", "infr_gguf_meta_count", "infr_gguf_meta_key", "infr_gguf_meta_type", "infr_gguf_meta_u64", "infr_gguf_meta_f64",
    "infr_gguf_meta_str", "infr_gguf_meta_array",
]


class BackendError(RuntimeError):
    """A failing C-ABI call: ``code`` is the INFR_E_* status, the text is infr_cuda_last_error()."""

    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code


class _GgufTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("ggml_type", C.c_uint32), ("dtype", C.c_int32), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 8),
                ("numel", C.c_uint64), ("nbytes", C.c_uint64), ("file_offset", C.c_uint64)]


class _Opts(C.Structure):
    _fields_ = [("device", C.c_int32), ("reference", C.c_int32), ("gemv_kernel", C.c_int32), ("mmq_kernel", C.c_int32), ("reserved", C.c_int32 * 4)]


class _Caps(C.Structure):
    _fields_ = [("name", C.c_char * 32), ("f16", C.c_int32), ("i8", C.c_int32), ("i8_dot", C.c_int32),
                ("integrated", C.c_int32), ("unified_memory", C.c_int32), ("decode_replay", C.c_int32),
                ("graph_input_inplace", C.c_int32), ("max_shared_memory_bytes", C.c_uint32),
                ("sm_count", C.c_uint32), ("total_memory_bytes", C.c_uint64), ("l2_bytes", C.c_uint64)]


class _TensorDecl(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("dtype", C.c_uint32), ("numel", C.c_uint64)]


class _OpDesc(C.Structure):
    _fields_ = [("tag", C.c_uint32), ("t", C.c_uint32 * 8), ("u", C.c_uint32 * 12), ("f", C.c_float * 4)]


class _MoeDesc(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("ne", C.c_uint32), ("n_expert", C.c_uint32), ("n_used", C.c_uint32),
                ("n_ff_exp", C.c_uint32), ("scale", C.c_float), ("norm_w", C.c_int32), ("router_dtype", C.c_int32),
                ("gate_dtype", C.c_int32), ("up_dtype", C.c_int32), ("down_dtype", C.c_int32),
                ("expert_lo", C.c_uint32), ("n_local", C.c_uint32)]


class _AttnDesc(C.Structure):
    _fields_ = [("rows", C.c_uint32), ("pos", C.c_uint32), ("n_head", C.c_uint32), ("n_kv", C.c_uint32), ("head_dim", C.c_uint32),
                ("scale", C.c_float), ("n_seq", C.c_uint32), ("reserved", C.c_uint32), ("seq_stride", C.c_uint64)]


class _Q8Out(C.Structure):
    _fields_ = [("qs", C.c_void_p), ("d", C.c_void_p), ("sums", C.c_void_p), ("sums16", C.c_void_p)]


class _GraphDesc(C.Structure):
    _fields_ = [("tensors", C.POINTER(_TensorDecl)), ("n_tensors", C.c_uint32),
                ("ops", C.POINTER(_OpDesc)), ("n_ops", C.c_uint32)]


_lib = None


def load_library() -> C.CDLL:
    """dlopen the in-tree library.  There is no fallback: a missing library is an error."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m infr_b200.build` (nvcc, sm_100a). "
            "infr_b200 has no CPU or PyTorch fallback.")
    L = C.CDLL(LIB_PATH)
    vp, u32, u64, i32, sz = C.c_void_p, C.c_uint32, C.c_uint64, C.c_int32, C.c_size_t
    sig = {
        "infr_cuda_create": (i32, [C.POINTER(_Opts), C.POINTER(vp)]),
        "infr_cuda_destroy": (None, [vp]),
        "infr_cuda_get_caps": (i32, [vp, C.POINTER(_Caps)]),
        "infr_cuda_last_error": (i32, [vp, C.c_char_p, sz]),
        "infr_cuda_alloc": (i32, [vp, sz, i32, C.POINTER(vp)]),
        "infr_cuda_alloc_uninit": (i32, [vp, sz, i32, C.POINTER(vp)]),
        "infr_cuda_free": (None, [vp, vp]),
        "infr_cuda_buf_len": (sz, [vp]),
        "infr_cuda_buf_device_ptr": (u64, [vp]),
        "infr_cuda_upload": (i32, [vp, vp, vp, sz]),
        "infr_cuda_upload_at": (i32, [vp, vp, sz, vp, sz]),
        "infr_cuda_download": (i32, [vp, vp, vp, sz]),
        "infr_cuda_copy": (i32, [vp, vp, vp, sz]),
        "infr_cuda_host_alloc": (i32, [vp, sz, C.POINTER(vp)]),
        "infr_cuda_host_free": (None, [vp, vp]),
        "infr_cuda_sync": (i32, [vp]),
        "infr_cuda_compile": (i32, [vp, C.POINTER(_GraphDesc), C.POINTER(vp)]),
        "infr_cuda_plan_free": (None, [vp, vp]),
        "infr_cuda_execute": (i32, [vp, vp, C.POINTER(vp), u32]),
        "infr_cuda_quantize_q8": (i32, [vp, i32, vp, u32, u32, vp, vp, vp, vp]),
        "infr_cuda_quantize_q8_1": (i32, [vp, vp, u32, u32, vp, vp, vp]),
        "infr_cuda_wrap": (i32, [vp, vp, sz, i32, C.POINTER(vp)]),
        "infr_cuda_stream": (vp, [vp]),
        "infr_cuda_comm_create": (i32, [vp, i32, i32, u32, C.POINTER(vp)]),
        "infr_cuda_comm_export": (i32, [vp, vp, vp]),
        "infr_cuda_comm_connect": (i32, [vp, vp, vp]),
        "infr_cuda_comm_connect_silent": (i32, [vp, vp, u32]),
        "infr_cuda_all_reduce_f32": (i32, [vp, vp, vp, u32]),
        "infr_cuda_comm_destroy": (None, [vp, vp]),
        "infr_cuda_gemv": (i32, [vp, i32, vp, u64, vp, vp, u32, u32, u32, i32]),
        "infr_cuda_gemv_q8": (i32, [vp, i32, vp, u64, vp, vp, vp, vp, vp, u32, u32, u32]),
        "infr_cuda_gemv_q8_pair": (i32, [vp, i32, vp, u64, vp, u32, vp, u64, vp, u32, vp, vp, vp, vp, u32, u32]),
        "infr_cuda_gemv_noalloc": (i32, [i32, vp, vp, vp, u32, u32, u32, vp, C.c_char_p, sz]),
        "infr_cuda_gemv_block_acc": (i32, [vp, i32, vp, u64, vp, vp, u32, u32]),
        "infr_cuda_linear": (i32, [vp, i32, vp, u64, vp, vp, u32, u32, u32, i32]),
        "infr_cuda_linear_pair": (i32, [vp, i32, vp, u64, vp, u32, vp, u64, vp, u32, vp, u32, u32, i32]),
        "infr_cuda_moe_ffn": (i32, [vp, C.POINTER(_MoeDesc), vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]),
        "infr_cuda_capture_begin": (i32, [vp]),
        "infr_cuda_capture_end": (i32, [vp, C.POINTER(vp)]),
        "infr_cuda_graph_launch": (i32, [vp, vp]),
        "infr_cuda_graph_free": (None, [vp, vp]),
        "infr_cuda_timer_start": (i32, [vp]),
        "infr_cuda_timer_stop": (i32, [vp, C.POINTER(C.c_float)]),
        "infr_cuda_flush_l2": (i32, [vp]),
        "infr_cuda_launch_count": (u64, [vp]),
        "infr_cuda_tensor_peak_i8": (i32, [vp, u32, u32, C.POINTER(C.c_float), C.POINTER(C.c_double)]),
        "infr_cuda_rms_norm": (i32, [vp, vp, vp, vp, u32, u32, C.c_float]),
        "infr_cuda_add_rms_norm": (i32, [vp, vp, vp, vp, vp, vp, u32, u32, C.c_float]),
        "infr_cuda_rope": (i32, [vp, vp, vp, vp, u32, u32, u32, u32, C.c_float, i32]),
        "infr_cuda_write_kv": (i32, [vp, vp, vp, u32, u32, u32]),
        "infr_cuda_attention": (i32, [vp, C.POINTER(_AttnDesc), vp, vp, vp, vp]),
        "infr_cuda_rope_write_kv": (i32, [vp, C.POINTER(_AttnDesc), C.c_float, i32, vp, vp, vp, vp, vp, vp]),
        "infr_cuda_gated_act": (i32, [vp, vp, vp, vp, u32, u32]),
        "infr_cuda_add": (i32, [vp, vp, vp, vp, u64]),
        "infr_cuda_argmax": (i32, [vp, vp, vp, u32, u32]),
        "infr_cuda_add_rms_norm_q8": (i32, [vp, vp, vp, vp, vp, u32, u32, C.c_float, C.POINTER(_Q8Out)]),
        "infr_cuda_gemv_q8_push": (i32, [vp, vp, i32, vp, u64, vp, vp, vp, vp, u32, u32, u32]),
        "infr_cuda_add_rms_norm_q8_pull": (i32, [vp, vp, vp, vp, vp, u32, u32, C.c_float, C.POINTER(_Q8Out)]),
        "infr_cuda_gated_act_q8": (i32, [vp, vp, vp, u32, u32, C.POINTER(_Q8Out)]),
        "infr_cuda_attention_q8": (i32, [vp, C.POINTER(_AttnDesc), vp, vp, vp, C.POINTER(_Q8Out)]),
        "infr_cuda_attention_seqpos": (i32, [vp, C.POINTER(_AttnDesc), vp, vp, vp, vp, vp]),
        "infr_cuda_attention_seqpos_q8": (i32, [vp, C.POINTER(_AttnDesc), vp, vp, vp, vp, C.POINTER(_Q8Out)]),
        "infr_cuda_attention_paged": (i32, [vp, C.POINTER(_AttnDesc), vp, vp, u32, u32, vp, vp, vp, vp, C.POINTER(_Q8Out)]),
        "infr_cuda_rope_write_kv_paged": (i32, [vp, C.POINTER(_AttnDesc), C.c_float, i32, vp, vp, vp, vp, vp, u32, u32, vp, vp]),
        "infr_gguf_open": (i32, [C.c_char_p, C.POINTER(vp), C.c_char_p, sz]),
        "infr_gguf_close": (None, [vp]),
        "infr_gguf_version": (u32, [vp]),
        "infr_gguf_alignment": (u64, [vp]),
        "infr_gguf_tensor_count": (u64, [vp]),
        "infr_gguf_tensor_at": (i32, [vp, u64, C.POINTER(_GgufTensor)]),
        "infr_gguf_find": (i32, [vp, C.c_char_p, C.POINTER(_GgufTensor)]),
        "infr_gguf_tensor_data": (vp, [vp, C.POINTER(_GgufTensor)]),
        "infr_gguf_meta_count": (u64, [vp]),
        "infr_gguf_meta_key": (C.c_char_p, [vp, u64]),
        "infr_gguf_meta_type": (i32, [vp, C.c_char_p]),
        "infr_gguf_meta_u64": (i32, [vp, C.c_char_p, C.POINTER(u64)]),
        "infr_gguf_meta_f64": (i32, [vp, C.c_char_p, C.POINTER(C.c_double)]),
        "infr_gguf_meta_str": (i32, [vp, C.c_char_p, C.POINTER(vp), C.POINTER(u64)]),
        "infr_gguf_meta_array": (i32, [vp, C.c_char_p, C.POINTER(u32), C.POINTER(u64), C.POINTER(vp)]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


@dataclass
class Capabilities:
    name: str
    f16: bool
    i8: bool
    i8_dot: bool
    integrated: bool
    unified_memory: bool
    decode_replay: bool
    graph_input_inplace: bool
    max_shared_memory_bytes: int
    sm_count: int
    total_memory_bytes: int
    l2_bytes: int


class Buffer:
    """Device buffer handle (`trait Buffer`, backend.rs:387-416).  Freed on close() / GC."""

    def __init__(self, be: "CudaBackend", handle: int, nbytes: int):
        self._be, self.handle, self.nbytes = be, handle, nbytes

    def len_bytes(self) -> int:
        return self.nbytes

    def device_ptr(self) -> int:
        return int(self._be.L.infr_cuda_buf_device_ptr(self.handle))

    def close(self):
        if self.handle and self._be.ctx:
            self._be.L.infr_cuda_free(self._be.ctx, self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Comm:
    """Peer-memory exchange group of one box (infr_cuda_comm_*): export() -> gather the handles of all ranks in rank
    order -> connect(handles) -> CudaBackend.all_reduce."""

    def __init__(self, be: "CudaBackend", handle, world: int):
        self._be, self.handle, self.world = be, handle, world

    def export(self) -> bytes:
        buf = (C.c_uint8 * 64)()
        self._be._check(self._be.L.infr_cuda_comm_export(self._be.ctx, self.handle, buf))
        return bytes(buf)

    def connect(self, handles: Sequence[bytes]):
        assert len(handles) == self.world and all(len(h) == 64 for h in handles)
        blob = (C.c_uint8 * (64 * self.world)).from_buffer_copy(b"".join(handles))
        self._be._check(self._be.L.infr_cuda_comm_connect(self._be.ctx, self.handle, blob))

    def connect_silent(self, spin_limit: int = 4096):
        """Failure-detection aid: peers that never answer (see infr_cuda_comm_connect_silent)."""
        self._be._check(self._be.L.infr_cuda_comm_connect_silent(self._be.ctx, self.handle, spin_limit))

    def close(self):
        """All ranks must have synchronised their last exchange and passed a host barrier before any rank closes."""
        if self.handle and self._be.ctx:
            self._be.L.infr_cuda_comm_destroy(self._be.ctx, self.handle)
        self.handle = None


class Graph:
    """Ordered op list over typed handles (crates/infr-core/src/graph.rs:1317-1460)."""

    def __init__(self):
        self.tensors: list[tuple[int, int, int]] = []
        self.ops: list[_OpDesc] = []

    def _decl(self, kind, dtype, numel) -> int:
        self.tensors.append((kind, dtype, int(numel)))
        return len(self.tensors) - 1

    def input(self, numel, dtype=F32):
        return self._decl(TK_INPUT, dtype, numel)

    def weight(self, numel, dtype):
        return self._decl(TK_WEIGHT, dtype, numel)

    def internal(self, numel, dtype=F32):
        return self._decl(TK_INTERNAL, dtype, numel)

    def output(self, numel, dtype=F32):
        return self._decl(TK_OUTPUT, dtype, numel)

    def linear(self, x, weight, dst, m, in_f, out_f, w_off=0):
        op = _OpDesc()
        op.tag = OP_LINEAR
        op.t[0], op.t[1], op.t[2] = x, weight, dst
        op.u[0], op.u[1], op.u[2], op.u[3] = m, in_f, out_f, w_off
        self.ops.append(op)

    def moe_ffn(self, x, router_x, router, gate_exps, up_exps, down_exps, dst, *, ne, n_expert, n_used,
                n_ff_exp, scale=1.0, norm_w=True, fused_gate_up=False, weight_before=False):
        op = _OpDesc()
        op.tag = OP_MOE_FFN
        for i, t in enumerate((x, router_x, router, gate_exps, up_exps, down_exps, dst)):
            op.t[i] = t
        for i, v in enumerate((ne, n_expert, n_used, n_ff_exp, int(norm_w), int(fused_gate_up),
                               int(weight_before), 0, 0)):
            op.u[i] = v
        op.f[0] = scale
        self.ops.append(op)


    def _op(self, tag, tensors, u=(), f=()):
        op = _OpDesc()
        op.tag = tag
        for i, t in enumerate(tensors):
            op.t[i] = t
        for i, v in enumerate(u):
            op.u[i] = int(v)
        for i, v in enumerate(f):
            op.f[i] = float(v)
        self.ops.append(op)

    # The remaining ops of a dense decode step, field for field with the Rust variants (graph.rs:141-896).
    def rms_norm(self, x, weight, dst, rows, dim, eps):
        self._op(OP_RMS_NORM, (x, weight, dst), (rows, dim), (eps,))

    def rope(self, x, positions, dst, rows, n_head, head_dim, rope_dim, theta, neox=False, x_stride=0, backward=False, freq_factors=None):
        self._op(OP_ROPE, (x, positions, dst), (rows, n_head, head_dim, rope_dim, x_stride, int(neox), int(backward), int(freq_factors is not None)), (theta,))

    def write_kv(self, src, cache, rows, row_stride, pos):
        self._op(OP_WRITE_KV, (src, cache), (rows, row_stride, pos))

    def attention(self, q, k_cache, v_cache, dst, rows, kv_len, n_head, n_kv, head_dim, scale, pos, mask=0, sinks=None):
        self._op(OP_ATTENTION, (q, k_cache, v_cache, dst), (rows, kv_len, n_head, n_kv, head_dim, mask, pos, int(sinks is not None)), (scale,))

    def gated_act(self, gate, up, dst, rows, nff, act=0, up_off=0, up_stride=0, gate_stride=0, gate_block_width=0, swiglu_clamp=None):
        self._op(OP_GATED_ACT, (gate, up, dst), (rows, nff, act, up_off, up_stride, gate_stride, gate_block_width, int(swiglu_clamp is not None)))

    def add(self, a, b, dst, n):
        self._op(OP_ADD, (a, b, dst), (n,))

    def argmax(self, x, dst, n, rows=1):
        self._op(OP_ARGMAX, (x, dst), (n, rows))

    def copy(self, src, src_off, dst, dst_off, n):
        self._op(OP_COPY, (src, dst), (src_off, dst_off, n))


class Plan:
    def __init__(self, be, handle):
        self._be, self.handle = be, handle

    def close(self):
        if self.handle and self._be.ctx:
            self._be.L.infr_cuda_plan_free(self._be.ctx, self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class CudaGraph:
    def __init__(self, be, handle):
        self._be, self.handle = be, handle

    def launch(self):
        self._be._check(self._be.L.infr_cuda_graph_launch(self._be.ctx, self.handle))

    def close(self):
        if self.handle and self._be.ctx:
            self._be.L.infr_cuda_graph_free(self._be.ctx, self.handle)
        self.handle = None


class CudaBackend:
    """`impl Backend for CudaBackend` over the C ABI."""

    def __init__(self, device: int = 0, reference: bool = False, gemv_kernel: int = 0, mmq_kernel: int = 0):
        """gemv_kernel / mmq_kernel: infr_cuda_opts' kernel selectors (0 = the default dispatch), used by the parity tests."""
        self.L = load_library()
        self.ctx = None
        opts = _Opts(device=device, reference=int(reference), gemv_kernel=int(gemv_kernel), mmq_kernel=int(mmq_kernel))
        ctx = C.c_void_p()
        rc = self.L.infr_cuda_create(C.byref(opts), C.byref(ctx))
        if rc != 0:
            buf = C.create_string_buffer(512)
            self.L.infr_cuda_last_error(None, buf, 512)
            raise BackendError(rc, buf.value.decode())
        self.ctx = ctx
        self.device = device
        self._pinned: list = []

    # ---- plumbing ----
    def _check(self, rc: int):
        if rc != 0:
            buf = C.create_string_buffer(1024)
            self.L.infr_cuda_last_error(self.ctx, buf, 1024)
            raise BackendError(rc, buf.value.decode())

    def close(self):
        if self.ctx:
            for p in self._pinned:
                self.L.infr_cuda_host_free(self.ctx, p)
            self._pinned = []
            self.L.infr_cuda_destroy(self.ctx)
            self.ctx = None

    def name(self) -> str:
        return self.capabilities().name

    def capabilities(self) -> Capabilities:
        c = _Caps()
        self._check(self.L.infr_cuda_get_caps(self.ctx, C.byref(c)))
        return Capabilities(c.name.decode(), bool(c.f16), bool(c.i8), bool(c.i8_dot), bool(c.integrated),
                            bool(c.unified_memory), bool(c.decode_replay), bool(c.graph_input_inplace),
                            c.max_shared_memory_bytes, c.sm_count, c.total_memory_bytes, c.l2_bytes)

    # ---- memory ----
    def alloc(self, nbytes: int, usage: int = USAGE_ACTIVATIONS) -> Buffer:
        h = C.c_void_p()
        self._check(self.L.infr_cuda_alloc(self.ctx, nbytes, usage, C.byref(h)))
        return Buffer(self, h, nbytes)

    def alloc_uninit(self, nbytes: int, usage: int = USAGE_WEIGHTS) -> Buffer:
        h = C.c_void_p()
        self._check(self.L.infr_cuda_alloc_uninit(self.ctx, nbytes, usage, C.byref(h)))
        return Buffer(self, h, nbytes)

    def wrap(self, device_ptr: int, nbytes: int, usage: int = USAGE_WEIGHTS) -> Buffer:
        """A handle over device memory the caller owns (e.g. ``tensor.data_ptr()``): nothing is allocated or
        copied and closing the handle leaves the memory alone.  The caller keeps the memory alive."""
        h = C.c_void_p()
        self._check(self.L.infr_cuda_wrap(self.ctx, C.c_void_p(device_ptr), nbytes, usage, C.byref(h)))
        return Buffer(self, h, nbytes)

    def comm_create(self, rank: int, world: int, max_floats: int) -> "Comm":
        h = C.c_void_p()
        self._check(self.L.infr_cuda_comm_create(self.ctx, rank, world, max_floats, C.byref(h)))
        return Comm(self, h, world)

    def all_reduce(self, comm: "Comm", data: Buffer, n: int):
        """In-place sum of n f32 over the comm's ranks, enqueued on the context's stream."""
        self._check(self.L.infr_cuda_all_reduce_f32(self.ctx, comm.handle, data.handle, n))

    def stream(self) -> int:
        """The context's cudaStream_t as an integer (0 = the default stream)."""
        return int(self.L.infr_cuda_stream(self.ctx) or 0)

    def upload(self, dst: Buffer, src: np.ndarray, offset: int = 0):
        src = np.ascontiguousarray(src)
        if offset:
            self._check(self.L.infr_cuda_upload_at(self.ctx, dst.handle, offset, src.ctypes.data, src.nbytes))
        else:
            self._check(self.L.infr_cuda_upload(self.ctx, dst.handle, src.ctypes.data, src.nbytes))

    def download(self, src: Buffer, dtype, count: Optional[int] = None) -> np.ndarray:
        dtype = np.dtype(dtype)
        n = src.nbytes // dtype.itemsize if count is None else count
        out = np.empty(n, dtype)
        self._check(self.L.infr_cuda_download(self.ctx, src.handle, out.ctypes.data, out.nbytes))
        return out

    def download_into(self, src: Buffer, dst: np.ndarray):
        self._check(self.L.infr_cuda_download(self.ctx, src.handle, dst.ctypes.data, dst.nbytes))

    def copy_buffer(self, src: Buffer, dst: Buffer, nbytes: int):
        self._check(self.L.infr_cuda_copy(self.ctx, src.handle, dst.handle, nbytes))

    def from_numpy(self, a: np.ndarray, usage: int = USAGE_ACTIVATIONS) -> Buffer:
        a = np.ascontiguousarray(a)
        b = self.alloc_uninit(max(a.nbytes, 4), usage)
        self.upload(b, a)
        return b

    def host_array(self, shape, dtype) -> np.ndarray:
        """A numpy array over page-locked host memory (freed when the backend closes)."""
        dtype = np.dtype(dtype)
        n = int(np.prod(shape))
        p = C.c_void_p()
        self._check(self.L.infr_cuda_host_alloc(self.ctx, n * dtype.itemsize, C.byref(p)))
        self._pinned.append(p)
        buf = (C.c_uint8 * (n * dtype.itemsize)).from_address(p.value)
        return np.frombuffer(buf, dtype=dtype, count=n).reshape(shape)

    def upload_raw(self, dst: Buffer, host_ptr: int, nbytes: int):
        self._check(self.L.infr_cuda_upload(self.ctx, dst.handle, host_ptr, nbytes))

    def download_raw(self, src: Buffer, host_ptr: int, nbytes: int):
        self._check(self.L.infr_cuda_download(self.ctx, src.handle, host_ptr, nbytes))

    def sync(self):
        self._check(self.L.infr_cuda_sync(self.ctx))

    # ---- graphs ----
    def compile(self, g: Graph) -> Plan:
        tens = (_TensorDecl * max(len(g.tensors), 1))()
        for i, (k, d, n) in enumerate(g.tensors):
            tens[i] = _TensorDecl(k, d, n)
        ops = (_OpDesc * max(len(g.ops), 1))(*g.ops)
        desc = _GraphDesc(tens, len(g.tensors), ops, len(g.ops))
        h = C.c_void_p()
        self._check(self.L.infr_cuda_compile(self.ctx, C.byref(desc), C.byref(h)))
        return Plan(self, h)

    def bind(self, bindings: dict[int, Buffer]):
        """The handle table of `execute` built once, for a plan that runs many times on the same buffers."""
        n = (max(bindings) + 1) if bindings else 0
        arr = (C.c_void_p * max(n, 1))()
        for i, b in bindings.items():
            arr[i] = b.handle
        return (arr, n, list(bindings.values()))  # the Buffers stay referenced as long as the table does

    def execute(self, plan: Plan, bindings):
        """bindings: {tensor id: Buffer}, or what bind() returned for such a dict."""
        arr, n, _ = bindings if isinstance(bindings, tuple) else self.bind(bindings)
        self._check(self.L.infr_cuda_execute(self.ctx, plan.handle, arr, n))

    # ---- direct kernels ----
    def quantize_q8(self, gran: int, x: Buffer, rows: int, k: int, qs: Buffer, d: Buffer, sums: Buffer,
                    sums16: Optional[Buffer] = None):
        self._check(self.L.infr_cuda_quantize_q8(self.ctx, gran, x.handle, rows, k, qs.handle, d.handle,
                                                 sums.handle, sums16.handle if sums16 else None))

    def quantize_q8_1(self, x: Buffer, rows: int, k: int, qs: Buffer, dact: Buffer, sact: Buffer):
        self._check(self.L.infr_cuda_quantize_q8_1(self.ctx, x.handle, rows, k, qs.handle, dact.handle, sact.handle))

    def gemv(self, dtype: int, w: Buffer, x: Buffer, y: Buffer, m: int, in_f: int, out_f: int,
             act: int = ACT_INT8, w_off: int = 0):
        self._check(self.L.infr_cuda_gemv(self.ctx, dtype, w.handle, w_off, x.handle, y.handle, m, in_f, out_f, act))

    def gemv_q8(self, dtype: int, w: Buffer, qs: Buffer, d: Buffer, sums: Buffer, sums16: Optional[Buffer],
                y: Buffer, m: int, in_f: int, out_f: int, w_off: int = 0):
        self._check(self.L.infr_cuda_gemv_q8(self.ctx, dtype, w.handle, w_off, qs.handle, d.handle, sums.handle,
                                             sums16.handle if sums16 else None, y.handle, m, in_f, out_f))

    def gemv_q8_pair(self, dtype: int, w1: Buffer, y1: Buffer, out_f1: int, w2: Buffer, y2: Buffer, out_f2: int, qs: Buffer, d: Buffer,
                     sums: Buffer, sums16: Optional[Buffer], m: int, in_f: int, w_off1: int = 0, w_off2: int = 0):
        """Two weights of one format against the same quantised rows (one launch for Q4_K)."""
        self._check(self.L.infr_cuda_gemv_q8_pair(self.ctx, dtype, w1.handle, w_off1, y1.handle, out_f1, w2.handle, w_off2, y2.handle, out_f2,
                                                  qs.handle, d.handle, sums.handle, sums16.handle if sums16 is not None else None, m, in_f))

    def linear(self, dtype: int, w: Buffer, x: Buffer, y: Buffer, m: int, in_f: int, out_f: int,
               act: int = ACT_INT8, w_off: int = 0):
        self._check(self.L.infr_cuda_linear(self.ctx, dtype, w.handle, w_off, x.handle, y.handle, m, in_f, out_f, act))

    def linear_pair(self, dtype: int, w1: Buffer, y1: Buffer, out_f1: int, w2: Buffer, y2: Buffer, out_f2: int, x: Buffer, m: int, in_f: int,
                    act: int = ACT_INT8, w_off1: int = 0, w_off2: int = 0):
        """Two Linears of one weight format on the same rows (rows quantised once; one launch for <= 8 rows of Q4_K)."""
        self._check(self.L.infr_cuda_linear_pair(self.ctx, dtype, w1.handle, w_off1, y1.handle, out_f1, w2.handle, w_off2, y2.handle, out_f2,
                                                 x.handle, m, in_f, act))

    def moe_ffn(self, x: Buffer, router_x: Buffer, router: Buffer, gate: Buffer, up: Buffer, down: Buffer, dst: Buffer, *,
                rows: int, ne: int, n_expert: int, n_used: int, n_ff_exp: int, scale: float = 1.0, norm_w: bool = True,
                wdt: int = Q4K, down_dt: Optional[int] = None, sel_ids: Optional[Buffer] = None, sel_w: Optional[Buffer] = None,
                logits: Optional[Buffer] = None, expert_lo: int = 0, n_local: int = 0):
        """Op::MoeFfn as a direct call.  wdt: format of the gate / up banks, down_dt: of the down bank (default wdt).
        n_local != 0: expert-parallel slice — the banks hold experts [expert_lo, expert_lo + n_local) and dst gets
        their contribution only (the ranks' dst add up)."""
        d = _MoeDesc(rows, ne, n_expert, n_used, n_ff_exp, scale, int(norm_w), F32, wdt, wdt, wdt if down_dt is None else down_dt,
                     expert_lo, n_local)
        h = lambda b: b.handle if b is not None else None
        self._check(self.L.infr_cuda_moe_ffn(self.ctx, C.byref(d), x.handle, router_x.handle, router.handle, gate.handle,
                                             up.handle, down.handle, dst.handle, h(sel_ids), h(sel_w), h(logits)))

    # ---- the other ops of a dense decode step (names and arguments follow the reference's Op variants) ----
    def rms_norm(self, x: Buffer, weight: Buffer, dst: Buffer, rows: int, dim: int, eps: float):
        self._check(self.L.infr_cuda_rms_norm(self.ctx, x.handle, weight.handle, dst.handle, rows, dim, eps))

    def add_rms_norm(self, a: Buffer, b: Buffer, sum_dst: Buffer, weight: Buffer, norm_dst: Buffer, rows: int, dim: int, eps: float):
        self._check(self.L.infr_cuda_add_rms_norm(self.ctx, a.handle, b.handle, sum_dst.handle, weight.handle, norm_dst.handle, rows, dim, eps))

    def rope(self, x: Buffer, positions: Buffer, dst: Buffer, rows: int, n_head: int, head_dim: int, rope_dim: int, theta: float,
             neox: bool = False):
        self._check(self.L.infr_cuda_rope(self.ctx, x.handle, positions.handle, dst.handle, rows, n_head, head_dim, rope_dim, theta, int(neox)))

    def write_kv(self, src: Buffer, cache: Buffer, rows: int, row_stride: int, pos: int):
        self._check(self.L.infr_cuda_write_kv(self.ctx, src.handle, cache.handle, rows, row_stride, pos))

    @staticmethod
    def _attn_desc(rows, pos, n_head, n_kv, head_dim, scale, n_seq, seq_stride):
        return _AttnDesc(rows, pos, n_head, n_kv, head_dim, scale, n_seq, 0, seq_stride)

    def attention(self, q: Buffer, k_cache: Buffer, v_cache: Buffer, dst: Buffer, *, rows: int, pos: int, n_head: int, n_kv: int,
                  head_dim: int, scale: float, n_seq: int = 1, seq_stride: int = 0, seq_pos: Optional[Buffer] = None):
        """seq_pos: int32 [n_seq] on the device, each sequence's own position (pos is then their maximum)."""
        d = self._attn_desc(rows, pos, n_head, n_kv, head_dim, scale, n_seq, seq_stride)
        if seq_pos is not None:
            self._check(self.L.infr_cuda_attention_seqpos(self.ctx, C.byref(d), seq_pos.handle, q.handle, k_cache.handle, v_cache.handle, dst.handle))
            return
        self._check(self.L.infr_cuda_attention(self.ctx, C.byref(d), q.handle, k_cache.handle, v_cache.handle, dst.handle))

    def rope_write_kv(self, q: Buffer, k: Buffer, v: Buffer, positions: Buffer, k_cache: Buffer, v_cache: Buffer, *, rows: int, pos: int,
                      n_head: int, n_kv: int, head_dim: int, theta: float, neox: bool = False, n_seq: int = 1, seq_stride: int = 0):
        d = self._attn_desc(rows, pos, n_head, n_kv, head_dim, 0.0, n_seq, seq_stride)
        self._check(self.L.infr_cuda_rope_write_kv(self.ctx, C.byref(d), theta, int(neox), q.handle, k.handle, v.handle, positions.handle,
                                                   k_cache.handle, v_cache.handle))

    def attention_paged(self, q: Buffer, k_pool: Buffer, v_pool: Buffer, block_table: Buffer, table_stride: int, n_pages: int, *, rows: int,
                        pos: int, n_head: int, n_kv: int, head_dim: int, scale: float, n_seq: int = 1, seq_pos: Optional[Buffer] = None,
                        dst: Optional[Buffer] = None, q8=None):
        """Attention over paged caches (pools of 128-row pages, a page table per sequence); q8 = (qs, d, sums, sums16)
        for the int8 form instead of dst."""
        d = self._attn_desc(rows, pos, n_head, n_kv, head_dim, scale, n_seq, 0)
        o = self._q8_out(*q8) if q8 is not None else None
        self._check(self.L.infr_cuda_attention_paged(self.ctx, C.byref(d), seq_pos.handle if seq_pos else None, block_table.handle, table_stride,
                                                     n_pages, q.handle, k_pool.handle, v_pool.handle, dst.handle if dst else None,
                                                     C.byref(o) if o is not None else None))

    def rope_write_kv_paged(self, q: Buffer, k: Buffer, v: Buffer, positions: Buffer, k_pool: Buffer, v_pool: Buffer, block_table: Buffer,
                            table_stride: int, n_pages: int, *, rows: int, pos: int, n_head: int, n_kv: int, head_dim: int, theta: float,
                            neox: bool = False, n_seq: int = 1):
        d = self._attn_desc(rows, pos, n_head, n_kv, head_dim, 0.0, n_seq, 0)
        self._check(self.L.infr_cuda_rope_write_kv_paged(self.ctx, C.byref(d), theta, int(neox), q.handle, k.handle, v.handle, positions.handle,
                                                         block_table.handle, table_stride, n_pages, k_pool.handle, v_pool.handle))

    def gated_act(self, gate: Buffer, up: Buffer, dst: Buffer, rows: int, nff: int):
        self._check(self.L.infr_cuda_gated_act(self.ctx, gate.handle, up.handle, dst.handle, rows, nff))

    def add(self, a: Buffer, b: Buffer, dst: Buffer, n: int):
        self._check(self.L.infr_cuda_add(self.ctx, a.handle, b.handle, dst.handle, n))

    @staticmethod
    def _q8_out(qs: Buffer, d: Buffer, sums: Buffer, sums16: Optional[Buffer]):
        return _Q8Out(qs.handle, d.handle, sums.handle, sums16.handle if sums16 else None)

    def add_rms_norm_q8(self, a: Buffer, b: Optional[Buffer], sum_dst: Optional[Buffer], weight: Buffer, rows: int, dim: int, eps: float,
                        qs: Buffer, d: Buffer, sums: Buffer, sums16: Optional[Buffer] = None):
        """RmsNorm (of a + b when b is given, the sum also written to sum_dst) ending in the activation quantiser."""
        o = self._q8_out(qs, d, sums, sums16)
        self._check(self.L.infr_cuda_add_rms_norm_q8(self.ctx, a.handle, b.handle if b else None, sum_dst.handle if sum_dst else None,
                                                     weight.handle, rows, dim, eps, C.byref(o)))

    def gemv_q8_push(self, comm: "Comm", dtype: int, w: Buffer, qs: Buffer, d: Buffer, sums: Buffer, sums16: Optional[Buffer], m: int, in_f: int,
                     out_f: int, w_off: int = 0):
        """gemv_q8 of a row-parallel Linear whose epilogue stores the partial result into every rank's staging (no buffer,
        no exchange kernel); add_rms_norm_q8_pull must follow."""
        self._check(self.L.infr_cuda_gemv_q8_push(self.ctx, comm.handle, dtype, w.handle, w_off, qs.handle, d.handle, sums.handle,
                                                  sums16.handle if sums16 is not None else None, m, in_f, out_f))

    def add_rms_norm_q8_pull(self, comm: "Comm", a: Buffer, sum_dst: Buffer, weight: Buffer, rows: int, dim: int, eps: float, qs: Buffer, d: Buffer,
                             sums: Buffer, sums16: Optional[Buffer] = None):
        """add_rms_norm_q8 with b = the sum over the ranks of the results pushed by gemv_q8_push."""
        o = self._q8_out(qs, d, sums, sums16)
        self._check(self.L.infr_cuda_add_rms_norm_q8_pull(self.ctx, comm.handle, a.handle, sum_dst.handle, weight.handle, rows, dim, eps, C.byref(o)))

    def gated_act_q8(self, gate: Buffer, up: Buffer, rows: int, nff: int, qs: Buffer, d: Buffer, sums: Buffer,
                     sums16: Optional[Buffer] = None):
        o = self._q8_out(qs, d, sums, sums16)
        self._check(self.L.infr_cuda_gated_act_q8(self.ctx, gate.handle, up.handle, rows, nff, C.byref(o)))

    def attention_q8(self, q: Buffer, k_cache: Buffer, v_cache: Buffer, qs: Buffer, d: Buffer, sums: Buffer, sums16: Optional[Buffer] = None, *,
                     rows: int, pos: int, n_head: int, n_kv: int, head_dim: int, scale: float, n_seq: int = 1, seq_stride: int = 0,
                     seq_pos: Optional[Buffer] = None):
        dsc = self._attn_desc(rows, pos, n_head, n_kv, head_dim, scale, n_seq, seq_stride)
        o = self._q8_out(qs, d, sums, sums16)
        if seq_pos is not None:
            self._check(self.L.infr_cuda_attention_seqpos_q8(self.ctx, C.byref(dsc), seq_pos.handle, q.handle, k_cache.handle, v_cache.handle, C.byref(o)))
            return
        self._check(self.L.infr_cuda_attention_q8(self.ctx, C.byref(dsc), q.handle, k_cache.handle, v_cache.handle, C.byref(o)))

    def argmax(self, x: Buffer, dst: Buffer, n: int, rows: int):
        self._check(self.L.infr_cuda_argmax(self.ctx, x.handle, dst.handle, n, rows))

    def gemv_block_acc(self, dtype: int, w: Buffer, x: Buffer, acc: Buffer, in_f: int, out_f: int, w_off: int = 0):
        self._check(self.L.infr_cuda_gemv_block_acc(self.ctx, dtype, w.handle, w_off, x.handle, acc.handle, in_f, out_f))

    # ---- capture / timing ----
    def capture_begin(self):
        self._check(self.L.infr_cuda_capture_begin(self.ctx))

    def capture_end(self) -> CudaGraph:
        h = C.c_void_p()
        self._check(self.L.infr_cuda_capture_end(self.ctx, C.byref(h)))
        return CudaGraph(self, h)

    def timer_start(self):
        self._check(self.L.infr_cuda_timer_start(self.ctx))

    def timer_stop(self) -> float:
        ms = C.c_float()
        self._check(self.L.infr_cuda_timer_stop(self.ctx, C.byref(ms)))
        return float(ms.value)

    def flush_l2(self):
        self._check(self.L.infr_cuda_flush_l2(self.ctx))

    def launch_count(self) -> int:
        return int(self.L.infr_cuda_launch_count(self.ctx))

    def tensor_peak_i8(self, n_batches: int = 64, launches: int = 20):
        """(milliseconds, int8 operations) of `launches` launches of the dense kind::i8 peak microbenchmark."""
        ms, ops = C.c_float(), C.c_double()
        self._check(self.L.infr_cuda_tensor_peak_i8(self.ctx, n_batches, launches, C.byref(ms), C.byref(ops)))
        return float(ms.value), float(ops.value)

    # ---- convenience used by tests: host arrays in, host array out, through the graph seam ----
    def run_linear(self, dtype: int, w_bytes: np.ndarray, x: np.ndarray, m: int, in_f: int, out_f: int,
                   w_off: int = 0, total_rows: Optional[int] = None) -> np.ndarray:
        """One-`Op::Linear` graph, the shape of infr_testkit::run_linear (testkit/src/lib.rs:314-337)."""
        rows = total_rows if total_rows is not None else out_f
        g = Graph()
        xid = g.input(m * in_f)
        wid = g.weight(rows * in_f, dtype)
        dst = g.output(m * out_f)
        g.linear(xid, wid, dst, m, in_f, out_f, w_off)
        plan = self.compile(g)
        xb = self.from_numpy(np.asarray(x, np.float32))
        wb = self.from_numpy(np.asarray(w_bytes, np.uint8), USAGE_WEIGHTS)
        ob = self.alloc(m * out_f * 4, USAGE_READBACK)
        self.execute(plan, {xid: xb, wid: wb, dst: ob})
        out = self.download(ob, np.float32).reshape(m, out_f)
        for b in (xb, wb, ob):
            b.close()
        plan.close()
        return out
