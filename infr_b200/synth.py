"""Seeded synthetic tensors in GGUF block formats (host side, numpy).

The benchmark configurations name shapes and distributions, not checkpoints: weights are drawn
fp32 N(0, 0.02) (or ternary) from a fixed seed and packed into Q4_K / Q6_K / Q2_0 blocks here, so
the CPU checker and the GPU consume byte-identical weight buffers.  Quantiser quality is
irrelevant to parity (both sides read the same bytes); the packers only have to emit valid blocks
with realistic scale/min statistics.

Block layouts (little endian) follow crates/infr-core/src/decode_spec.rs:327 (Q4_K), :331 (Q6_K),
:358 (Q2_0) and the decode in crates/infr-gguf/src/dequant.rs:311-331, :361-385, :1003-1019.
"""
from __future__ import annotations

import numpy as np

F32, Q4K, Q6K, Q2_0 = 0, 12, 14, 27
BLOCK_ELEMS = {F32: 1, Q4K: 256, Q6K: 256, Q2_0: 64}
BLOCK_BYTES = {F32: 4, Q4K: 144, Q6K: 210, Q2_0: 18}
DTYPE_NAMES = {F32: "f32", Q4K: "q4_k", Q6K: "q6_k", Q2_0: "q2_0"}


def row_bytes(dtype: int, in_f: int) -> int:
    be = BLOCK_ELEMS[dtype]
    if in_f % be:
        raise ValueError(f"in_f={in_f} is not a whole number of {be}-element blocks")
    return in_f // be * BLOCK_BYTES[dtype]


def rng(seed: int) -> np.random.Generator:
    """Counter-based generator (Philox) so a seed reproduces the same stream on any host."""
    return np.random.Generator(np.random.Philox(seed))


def normal(seed: int, shape, sigma: float = 1.0) -> np.ndarray:
    return (rng(seed).standard_normal(shape, dtype=np.float32) * np.float32(sigma)).astype(np.float32)


def _round_half_away(v: np.ndarray) -> np.ndarray:
    return np.sign(v) * np.floor(np.abs(v) + 0.5)


# --------------------------------------------------------------------------------------------
def quantize_q4k(w: np.ndarray) -> np.ndarray:
    """fp32 [..., k] (k % 256 == 0) -> raw Q4_K bytes, 144 per 256 values.

    Per 32-value sub-block: min = min(x, 0), scale = (max - min) / 15; super-block d = max scale/63,
    dmin = max(-min)/63 (both stored f16); 6-bit sc/m; codes re-quantised against the f16-rounded
    scales the decoder will reconstruct: q = clamp(round((x + dmin*m) / (d*sc)), 0, 15).
    """
    x = np.ascontiguousarray(w, dtype=np.float32).reshape(-1, 8, 32)
    nb = x.shape[0]
    lo = np.minimum(x.min(axis=2), 0.0)
    hi = np.maximum(x.max(axis=2), 0.0)
    sub_sc = (hi - lo) / np.float32(15.0)
    d = (sub_sc.max(axis=1) / np.float32(63.0)).astype(np.float16)
    dmin = ((-lo).max(axis=1) / np.float32(63.0)).astype(np.float16)
    df, dmf = d.astype(np.float32), dmin.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df[:, None] > 0, _round_half_away(sub_sc / df[:, None]), 0)
        mn = np.where(dmf[:, None] > 0, _round_half_away(-lo / dmf[:, None]), 0)
    sc = np.clip(sc, 0, 63).astype(np.uint8)
    mn = np.clip(mn, 0, 63).astype(np.uint8)
    scale = df[:, None] * sc.astype(np.float32)
    minv = dmf[:, None] * mn.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(scale[:, :, None] > 0, (x + minv[:, :, None]) / scale[:, :, None], 0)
    q = np.clip(_round_half_away(q), 0, 15).astype(np.uint8)

    out = np.zeros((nb, 144), dtype=np.uint8)
    out[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
    out[:, 2:4] = dmin.view(np.uint8).reshape(nb, 2)
    for k in range(4):
        out[:, 4 + k] = (sc[:, k] & 63) | (((sc[:, 4 + k] >> 4) & 3) << 6)
        out[:, 8 + k] = (mn[:, k] & 63) | (((mn[:, 4 + k] >> 4) & 3) << 6)
        out[:, 12 + k] = (sc[:, 4 + k] & 0xF) | ((mn[:, 4 + k] & 0xF) << 4)
    for pair in range(4):
        out[:, 16 + pair * 32:16 + pair * 32 + 32] = q[:, 2 * pair, :] | (q[:, 2 * pair + 1, :] << 4)
    return out.reshape(-1)


def quantize_q6k(w: np.ndarray) -> np.ndarray:
    """fp32 [..., k] (k % 256 == 0) -> raw Q6_K bytes, 210 per 256 values.

    Per 16-value group: s = amax/31; super-block d = max s / 127 (f16); int8 sc = round(s/d);
    code = clamp(round(x / (d*sc)), -32, 31) + 32.
    """
    x = np.ascontiguousarray(w, dtype=np.float32).reshape(-1, 16, 16)
    nb = x.shape[0]
    s = np.abs(x).max(axis=2) / np.float32(31.0)
    d = (s.max(axis=1) / np.float32(127.0)).astype(np.float16)
    df = d.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        sc = np.where(df[:, None] > 0, _round_half_away(s / df[:, None]), 0)
    sc = np.clip(sc, 0, 127).astype(np.int8)
    scale = df[:, None] * sc.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(scale[:, :, None] > 0, x / scale[:, :, None], 0)
    q = (np.clip(_round_half_away(q), -32, 31) + 32).astype(np.uint8).reshape(nb, 2, 4, 32)
    out = np.zeros((nb, 210), dtype=np.uint8)
    for h in range(2):
        e0, e1, e2, e3 = (q[:, h, k, :] for k in range(4))
        out[:, h * 64:h * 64 + 32] = (e0 & 0xF) | ((e2 & 0xF) << 4)
        out[:, h * 64 + 32:h * 64 + 64] = (e1 & 0xF) | ((e3 & 0xF) << 4)
        out[:, 128 + h * 32:128 + h * 32 + 32] = (e0 >> 4) | ((e1 >> 4) << 2) | ((e2 >> 4) << 4) | ((e3 >> 4) << 6)
    out[:, 192:208] = sc.view(np.uint8)
    out[:, 208:210] = d.view(np.uint8).reshape(nb, 2)
    return out.reshape(-1)


def pack_q2_0(tern: np.ndarray, d: np.ndarray) -> np.ndarray:
    """Ternary values in {-1,0,+1} [..., k] (k % 64 == 0) + one scale per 64 -> raw Q2_0 bytes.

    Element j of a block sits in byte j/4 at bit 2*(j%4); code = value + 1.
    """
    t = (np.ascontiguousarray(tern).reshape(-1, 16, 4) + 1).astype(np.uint8)
    nb = t.shape[0]
    out = np.zeros((nb, 18), dtype=np.uint8)
    out[:, 0:2] = np.ascontiguousarray(d, dtype=np.float16).reshape(nb).view(np.uint8).reshape(nb, 2)
    out[:, 2:18] = t[:, :, 0] | (t[:, :, 1] << 2) | (t[:, :, 2] << 4) | (t[:, :, 3] << 6)
    return out.reshape(-1)


# --------------------------------------------------------------------------------------------
def weight(dtype: int, out_f: int, in_f: int, seed: int, sigma: float = 0.02) -> np.ndarray:
    """Raw bytes of a seeded [out_f, in_f] weight in `dtype` (row-major, whole blocks per row)."""
    if dtype == Q2_0:
        g = rng(seed)
        u = g.random((out_f, in_f), dtype=np.float32)
        tern = np.where(u < 0.25, -1, np.where(u < 0.75, 0, 1)).astype(np.int8)
        d = (np.float32(sigma) * (np.float32(0.5) + g.random(out_f * in_f // 64, dtype=np.float32)))
        return pack_q2_0(tern, d)
    w = normal(seed, (out_f, in_f), sigma)
    if dtype == Q4K:
        return quantize_q4k(w)
    if dtype == Q6K:
        return quantize_q6k(w)
    if dtype == F32:
        return w.reshape(-1).view(np.uint8)
    raise ValueError(f"unsupported dtype code {dtype}")


def random_blocks(dtype: int, n_elem: int, seed: int) -> np.ndarray:
    """Random but valid blocks (uniform payload bytes, sane f16 scales) without an fp32 detour.

    Used where only the byte volume and validity matter (multi-gigabyte stacks for timing).
    """
    be, bb = BLOCK_ELEMS[dtype], BLOCK_BYTES[dtype]
    nb = n_elem // be
    g = rng(seed)
    raw = g.integers(0, 256, size=(nb, bb), dtype=np.uint8)
    d = (np.float32(2e-3) * (np.float32(0.5) + g.random(nb, dtype=np.float32))).astype(np.float16)
    if dtype == Q4K:
        raw[:, 0:2] = d.view(np.uint8).reshape(nb, 2)
        raw[:, 2:4] = (d * np.float16(0.5)).view(np.uint8).reshape(nb, 2)
    elif dtype == Q6K:
        raw[:, 208:210] = (d * np.float16(0.25)).view(np.uint8).reshape(nb, 2)
    elif dtype == Q2_0:
        raw[:, 0:2] = (d * np.float16(10)).view(np.uint8).reshape(nb, 2)
    return raw.reshape(-1)
