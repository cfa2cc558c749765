"""GGUF files on the weight side of the backend: `GgufFile` wraps the library's reader (infr_gguf_*, the counterpart
of Gguf::open / tensor_bytes / Metadata in crates/infr-gguf/src/lib.rs:82-145, :476, :893-930), `load_llama` turns a
Llama-family file into the device buffers a `DecodeStep` runs on — every weight goes mapping -> device in one upload,
no host copy in between (the loader path of the reference: mmap, then the backend's upload of the raw blocks).

Tensor names and metadata keys are the llama.cpp conventions the reference reads
(crates/infr-llama/src/seam/runner.rs weights: `blk.N.attn_q.weight` ..., `token_embd.weight`, `output_norm.weight`,
`output.weight`; hyper-parameters `<arch>.block_count`, `.embedding_length`, `.attention.head_count[_kv]`,
`.feed_forward_length`, `.rope.freq_base`, `.attention.layer_norm_rms_epsilon`)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import (F16, Q2_0, Q4K, Q6K, USAGE_ACTIVATIONS, USAGE_WEIGHTS, BackendError, _GgufTensor, load_library)

GGML_F32, GGML_F16, GGML_Q4_K, GGML_Q6_K, GGML_Q2_0 = 0, 1, 12, 14, 42


@dataclass
class GgufTensor:
    name: str
    ggml_type: int
    dtype: int          # the backend's dtype code, or -1 when the backend does not run this type
    dims: Tuple[int, ...]  # dims[0] is the fastest-varying axis (columns)
    numel: int
    nbytes: int
    file_offset: int
    _raw: _GgufTensor = None


class GgufFile:
    """A mapped GGUF file.  Tensor data is exposed as read-only numpy views of the mapping (valid until close())."""

    def __init__(self, path: str):
        self.L = load_library()
        h = C.c_void_p()
        err = C.create_string_buffer(512)
        rc = self.L.infr_gguf_open(str(path).encode(), C.byref(h), err, len(err))
        if rc != 0:
            raise BackendError(rc, err.value.decode(errors="replace"))
        self.h = h
        self.version = int(self.L.infr_gguf_version(h))
        self.alignment = int(self.L.infr_gguf_alignment(h))
        self.tensors: Dict[str, GgufTensor] = {}
        for i in range(int(self.L.infr_gguf_tensor_count(h))):
            t = _GgufTensor()
            if self.L.infr_gguf_tensor_at(h, i, C.byref(t)) != 0:
                raise BackendError(-1, f"GGUF: tensor {i}")
            name = t.name.decode()
            self.tensors[name] = GgufTensor(name, int(t.ggml_type), int(t.dtype), tuple(int(t.dims[d]) for d in range(t.n_dims)), int(t.numel),
                                            int(t.nbytes), int(t.file_offset), t)

    def close(self):
        if self.h:
            self.L.infr_gguf_close(self.h)
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    # ---- metadata
    def keys(self) -> List[str]:
        return [self.L.infr_gguf_meta_key(self.h, i).decode() for i in range(int(self.L.infr_gguf_meta_count(self.h)))]

    def meta(self, key: str, default=None):
        """The value of a metadata key: int, float, bool, str, a numpy array (numeric arrays) or the element count
        (arrays of strings / arrays); `default` when the key is absent."""
        k = key.encode()
        t = int(self.L.infr_gguf_meta_type(self.h, k))
        if t < 0:
            return default
        if t in (0, 1, 2, 3, 4, 5, 10, 11):
            if t in (1, 3, 5, 11):
                f = C.c_double()
                self.L.infr_gguf_meta_f64(self.h, k, C.byref(f))
                return int(f.value)
            v = C.c_uint64()
            self.L.infr_gguf_meta_u64(self.h, k, C.byref(v))
            return int(v.value)
        if t == 7:
            v = C.c_uint64()
            self.L.infr_gguf_meta_u64(self.h, k, C.byref(v))
            return bool(v.value)
        if t in (6, 12):
            f = C.c_double()
            self.L.infr_gguf_meta_f64(self.h, k, C.byref(f))
            return float(f.value)
        if t == 8:
            p, n = C.c_void_p(), C.c_uint64()
            self.L.infr_gguf_meta_str(self.h, k, C.byref(p), C.byref(n))
            return C.string_at(p, n.value).decode(errors="replace")
        et, n, p = C.c_uint32(), C.c_uint64(), C.c_void_p()
        self.L.infr_gguf_meta_array(self.h, k, C.byref(et), C.byref(n), C.byref(p))
        np_types = {0: np.uint8, 1: np.int8, 2: np.uint16, 3: np.int16, 4: np.uint32, 5: np.int32, 6: np.float32, 7: np.uint8, 10: np.uint64,
                    11: np.int64, 12: np.float64}
        if et.value in np_types and p.value:
            dt = np.dtype(np_types[et.value])
            return np.frombuffer(C.string_at(p, n.value * dt.itemsize), dt).copy()
        return int(n.value)

    # ---- tensors
    def data(self, name: str) -> np.ndarray:
        """The tensor's bytes as a uint8 view of the mapping (no copy)."""
        t = self.tensors[name]
        p = self.L.infr_gguf_tensor_data(self.h, C.byref(t._raw))
        if not p:
            raise BackendError(-1, f"GGUF: tensor '{name}' has no data in the mapping")
        buf = (C.c_uint8 * t.nbytes).from_address(p)
        a = np.frombuffer(buf, np.uint8)
        a.flags.writeable = False
        return a

    def upload(self, be, name: str, dst=None, dst_offset: int = 0, usage: int = USAGE_WEIGHTS):
        """Sends the tensor from the mapping to the device: into `dst` at `dst_offset`, or into a new buffer."""
        t = self.tensors[name]
        p = self.L.infr_gguf_tensor_data(self.h, C.byref(t._raw))
        if not p:
            raise BackendError(-1, f"GGUF: tensor '{name}' has no data in the mapping")
        if dst is None:
            dst = be.alloc_uninit(max(t.nbytes, 4), usage)
        be._check(be.L.infr_cuda_upload_at(be.ctx, dst.handle, dst_offset, p, t.nbytes))
        return dst


_BLOCK = {GGML_Q4_K: (256, 144), GGML_Q6_K: (256, 210), GGML_Q2_0: (64, 18)}


def dequant_blocks(ggml_type: int, raw: np.ndarray) -> np.ndarray:
    """f32 values of whole Q4_K / Q6_K / Q2_0 blocks (crates/infr-gguf/src/dequant.rs:11-51, the factored decode of
    :311-331 and :361-385 and the codebook arm :1003-1019): out = (d * sc) * code + (dmin * -m), every product and the
    sum rounded to f32 on its own.  Host side only: one embedding row per token of a file whose token_embd is
    quantised (what a Q4_K_M file ships); the Linears never leave the device."""
    be, bb = _BLOCK[ggml_type]
    blk = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1, bb)
    nb = blk.shape[0]
    f32 = np.float32
    out = np.empty((nb, be), f32)
    if ggml_type == GGML_Q4_K:
        d = blk[:, 0:2].copy().view(np.float16).astype(f32)      # [nb, 1]
        dmin = blk[:, 2:4].copy().view(np.float16).astype(f32)
        sc_b, qs = blk[:, 4:16].astype(np.int32), blk[:, 16:144]

        def k4(j):  # get_scale_min_k4 (dequant.rs:73-83)
            if j < 4:
                return sc_b[:, j] & 63, sc_b[:, j + 4] & 63
            return (sc_b[:, j + 4] & 0xF) | ((sc_b[:, j - 4] >> 6) << 4), (sc_b[:, j + 4] >> 4) | ((sc_b[:, j] >> 6) << 4)
        for j in range(4):
            for half, codes in ((0, qs[:, 32 * j:32 * j + 32] & 0xF), (1, qs[:, 32 * j:32 * j + 32] >> 4)):
                sc, m = k4(2 * j + half)
                s = d * sc.astype(f32)[:, None]
                n = dmin * (-m).astype(f32)[:, None]
                out[:, 64 * j + 32 * half:64 * j + 32 * half + 32] = s * codes.astype(f32) + n
        return out.reshape(-1)
    if ggml_type == GGML_Q6_K:
        ql, qh = blk[:, 0:128], blk[:, 128:192]
        scales = blk[:, 192:208].copy().view(np.int8).astype(np.int32)
        d = blk[:, 208:210].copy().view(np.float16).astype(f32)
        for half in range(2):
            lo0, lo1 = ql[:, 64 * half:64 * half + 32], ql[:, 64 * half + 32:64 * half + 64]
            h = qh[:, 32 * half:32 * half + 32]
            codes = [(lo0 & 0xF) | ((h & 3) << 4), (lo1 & 0xF) | (((h >> 2) & 3) << 4), (lo0 >> 4) | (((h >> 4) & 3) << 4),
                     (lo1 >> 4) | (((h >> 6) & 3) << 4)]
            for k in range(4):
                s16 = np.repeat(scales[:, 8 * half + 2 * k:8 * half + 2 * k + 2], 16, axis=1)  # the scale of l is scales[is + 2k], is = l / 16
                sc = d * s16.astype(f32)
                mn = d * (-32 * s16).astype(f32)
                out[:, 128 * half + 32 * k:128 * half + 32 * k + 32] = sc * codes[k].astype(f32) + mn
        return out.reshape(-1)
    if ggml_type == GGML_Q2_0:
        d = blk[:, 0:2].copy().view(np.float16).astype(f32)
        qs = blk[:, 2:18]
        codes = np.stack([(qs >> (2 * k)) & 3 for k in range(4)], axis=2).reshape(nb, 64).astype(np.int32)  # element j: byte j / 4, bits 2 (j % 4)
        out[:] = (codes - 1).astype(f32) * d
        return out.reshape(-1)
    raise BackendError(-2, f"GGUF: no host decode for ggml type {ggml_type}")


def _f32_row(g: GgufFile, name: str, row: int) -> np.ndarray:
    """One row of a tensor as f32 (the host-side embedding lookup: the backend reports no embed_gather): F32, F16, or
    the three block formats this backend runs, decoded on the host."""
    t = g.tensors[name]
    cols = t.dims[0]
    raw = g.data(name)
    if t.ggml_type == GGML_F32:
        return raw.view(np.float32)[row * cols:(row + 1) * cols].copy()
    if t.ggml_type == GGML_F16:
        return raw.view(np.float16)[row * cols:(row + 1) * cols].astype(np.float32)
    if t.ggml_type in _BLOCK:
        be, bb = _BLOCK[t.ggml_type]
        if cols % be:
            raise BackendError(-1, f"GGUF: '{name}' has rows of {cols} elements, not whole {be}-element blocks")
        bpr = cols // be * bb
        return dequant_blocks(t.ggml_type, raw[row * bpr:(row + 1) * bpr])
    raise BackendError(-2, f"GGUF: embedding lookup from ggml type {t.ggml_type} is not built (F32, F16, Q4_K, Q6_K and Q2_0 are)")


@dataclass
class LoadedLlama:
    shape: object          # LlamaShape
    layers: list           # per layer: name -> Buffer, plus "dtypes": name -> backend dtype code
    out_norm: object
    head: object
    head_dtype: int
    fused_qkv: list        # per layer: (Buffer holding wq | wk | wv rows back to back, dtype) or None
    gguf: GgufFile

    def embed(self, token_ids) -> np.ndarray:
        """Rows of token_embd for the ids, f32 [n, hidden]."""
        return np.stack([_f32_row(self.gguf, "token_embd.weight", int(t)) for t in token_ids])


_LAYER_TENSORS = [("wq", "attn_q"), ("wk", "attn_k"), ("wv", "attn_v"), ("wo", "attn_output"), ("gate", "ffn_gate"), ("up", "ffn_up"),
                  ("down", "ffn_down")]


def load_llama(be, path: str) -> LoadedLlama:
    """Reads a Llama-family GGUF (no biases, no QK norm) whose Linears are Q4_K / Q6_K / Q2_0 and uploads it."""
    from .decode import LlamaShape
    g = GgufFile(path)
    arch = g.meta("general.architecture", "llama")
    need = lambda k: _need(g, f"{arch}.{k}")
    n_layer, hidden, n_head = need("block_count"), need("embedding_length"), need("attention.head_count")
    n_kv = g.meta(f"{arch}.attention.head_count_kv", n_head)
    ffn = need("feed_forward_length")
    head_dim = g.meta(f"{arch}.attention.key_length", hidden // n_head)
    emb = g.tensors.get("token_embd.weight")
    if emb is None:
        raise BackendError(-1, "GGUF: no token_embd.weight")
    vocab = emb.dims[1]
    shape = LlamaShape(n_layer=n_layer, hidden=hidden, n_head=n_head, n_kv=n_kv, head_dim=head_dim, ffn=ffn, vocab=vocab,
                       theta=float(g.meta(f"{arch}.rope.freq_base", 10000.0)), eps=float(g.meta(f"{arch}.attention.layer_norm_rms_epsilon", 1e-5)))
    def weight(name):
        t = g.tensors.get(name)
        if t is None:
            raise BackendError(-1, f"GGUF: no tensor '{name}'")
        if t.dtype not in (Q4K, Q6K, Q2_0):
            raise BackendError(-2, f"GGUF: '{name}' has ggml type {t.ggml_type}; this backend runs Q4_K, Q6_K and Q2_0 Linears")
        return t
    def norm(name):
        t = g.tensors.get(name)
        if t is None or t.ggml_type != GGML_F32:
            raise BackendError(-1, f"GGUF: norm weight '{name}' missing or not F32")
        return g.upload(be, name, usage=USAGE_ACTIVATIONS)
    layers, fused = [], []
    for li in range(n_layer):
        L, dts = {}, {}
        for short, long in _LAYER_TENSORS:
            t = weight(f"blk.{li}.{long}.weight")
            L[short] = g.upload(be, t.name)
            dts[short] = t.dtype
        L["dtypes"] = dts
        L["attn_norm"] = norm(f"blk.{li}.attn_norm.weight")
        L["ffn_norm"] = norm(f"blk.{li}.ffn_norm.weight")
        layers.append(L)
        # q | k | v rows back to back in one buffer where the three share a format: the `w_off` slices of a fused-QKV
        # Linear (the reference does this at decode, seam/runner.rs:3445-3461)
        if dts["wq"] == dts["wk"] == dts["wv"]:
            names = [f"blk.{li}.{n}.weight" for n in ("attn_q", "attn_k", "attn_v")]
            total = sum(g.tensors[n].nbytes for n in names)
            buf, off = be.alloc_uninit(total, USAGE_WEIGHTS), 0
            for n in names:
                g.upload(be, n, buf, off)
                off += g.tensors[n].nbytes
            fused.append((buf, dts["wq"]))
        else:
            fused.append(None)
    out_norm = norm("output_norm.weight")
    head_name = "output.weight" if "output.weight" in g.tensors else "token_embd.weight"  # tied embeddings
    ht = weight(head_name)
    head = g.upload(be, head_name)
    return LoadedLlama(shape, layers, out_norm, head, ht.dtype, fused, g)


def _need(g: GgufFile, key: str):
    v = g.meta(key)
    if v is None:
        raise BackendError(-1, f"GGUF: metadata key '{key}' is missing")
    return v
