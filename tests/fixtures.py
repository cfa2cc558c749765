"""Deterministic inputs restated from the reference's own tests (generators only, no outputs).

* det_bytes / det_x        — crates/infr-cpu/src/kernels.rs:6611-6624 (64-bit LCG)
* lcg_bytes / gen_f32 / synth_weight / case_inputs
                           — crates/infr-testkit/src/lib.rs:49-64, :106-123, :290-310
"""
import numpy as np

M64 = (1 << 64) - 1
Q4K, Q6K, Q2_0 = 12, 14, 27
BLOCK = {Q4K: (256, 144), Q6K: (256, 210), Q2_0: (64, 18)}
# position of each dtype in WEIGHT_QUANTS (crates/infr-core/src/decode_spec.rs:255-280)
WEIGHT_QUANTS_INDEX = {Q4K: 7, Q6K: 9, Q2_0: 21}
# synth_scales (crates/infr-testkit/src/lib.rs:73-95)
SYNTH_SCALES = {Q4K: (0.05, 0.10), Q6K: (0.03, 0.0), Q2_0: (0.05, 0.0)}
D_SLOT = {Q4K: 0, Q6K: 208, Q2_0: 0}
MIN_SLOT = {Q4K: 2}


def _lcg64(seed):
    return (seed * 6364136223846793005 + 1442695040888963407) & M64


def det_bytes(n, seed):
    out = np.empty(n, np.uint8)
    for i in range(n):
        seed = _lcg64(seed)
        out[i] = (seed >> 33) & 0xFF
    return out


def det_x(n, seed):
    out = np.empty(n, np.float32)
    for i in range(n):
        seed = _lcg64(seed)
        out[i] = np.float32(np.float32(seed >> 40) / np.float32(1 << 24)) * np.float32(2.0) - np.float32(1.0)
    return out


def put_f16(buf, off, v):
    buf[off:off + 2] = np.array([v], np.float32).astype(np.float16).view(np.uint8)


def lcg_bytes(seed, n):
    out = np.empty(n, np.uint8)
    seed &= 0xFFFFFFFF
    for i in range(n):
        seed = (seed * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = (seed >> 16) & 0xFF
    return out


def gen_f32(n, salt):
    i = np.arange(n, dtype=np.int64)
    return (((i * 13 + salt) % 29).astype(np.float32) - np.float32(14.0)) * np.float32(0.05)


def synth_weight(dtype, n_elem, seed):
    be, bb = BLOCK[dtype]
    nblk = n_elem // be
    d, mn = SYNTH_SCALES[dtype]
    out = np.empty(nblk * bb, np.uint8)
    for b in range(nblk):
        blk = lcg_bytes(seed ^ b, bb)
        put_f16(blk, D_SLOT[dtype], d)
        if dtype in MIN_SLOT:
            put_f16(blk, MIN_SLOT[dtype], mn)
        out[b * bb:(b + 1) * bb] = blk
    return out


def case_inputs(dtype, m, in_f, out_f, seed):
    """(weight bytes, activations) of a LinearCase."""
    return synth_weight(dtype, out_f * in_f, seed), gen_f32(m * in_f, seed ^ 0x9E37)


def weight_quant_case_seed(dtype):
    return 0x201 + WEIGHT_QUANTS_INDEX[dtype]


def rel_l2(got, want):
    got = np.asarray(got, np.float64).ravel()
    want = np.asarray(want, np.float64).ravel()
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))
