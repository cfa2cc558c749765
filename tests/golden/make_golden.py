"""Regenerates tests/golden/kquant_decode.npz.

The reference's decode of Q4_K / Q6_K follows the published GGUF block formats.  The reference
itself is Rust and cannot be run where this repository is built, so the expected values here come
from an INDEPENDENT implementation of the same published formats: the numpy dequantiser of the
`gguf` Python package (llama.cpp's own reader).  Inputs are the deterministic blocks the
reference's kernel tests use (64-bit LCG payload with patched f16 scales,
crates/infr-cpu/src/kernels.rs:6611-6681) plus the patterned blocks of
crates/infr-gguf/src/dequant.rs:1170-1199.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from fixtures import det_bytes, put_f16  # noqa: E402


def main():
    from gguf import GGMLQuantizationType as T
    from gguf import quants

    out = {}
    # kernels.rs q4k_dot_matches_dequant_reference: 3 blocks, seed 1, d=0.05 dmin=0.015
    w = det_bytes(3 * 144, 1)
    for k in range(3):
        put_f16(w, k * 144, 0.05)
        put_f16(w, k * 144 + 2, 0.015)
    out["q4k_lcg_bytes"] = w
    out["q4k_lcg_f32"] = quants.dequantize(w.reshape(3, 144), T.Q4_K).astype(np.float32).ravel()
    # kernels.rs q6k_dot_matches_dequant_reference: 3 blocks, seed 3, d=0.04
    w = det_bytes(3 * 210, 3)
    for k in range(3):
        put_f16(w, k * 210 + 208, 0.04)
    out["q6k_lcg_bytes"] = w
    out["q6k_lcg_f32"] = quants.dequantize(w.reshape(3, 210), T.Q6_K).astype(np.float32).ravel()
    # dequant.rs affine_single_pass_bit_identical_q4k / _q6k patterned blocks
    w = ((np.arange(288) * 37 + 11) & 0xFF).astype(np.uint8)
    for b in range(2):
        put_f16(w, b * 144, 0.375)
        put_f16(w, b * 144 + 2, -0.125)
    out["q4k_pat_bytes"] = w
    out["q4k_pat_f32"] = quants.dequantize(w.reshape(2, 144), T.Q4_K).astype(np.float32).ravel()
    w = ((np.arange(420) * 53 + 7) & 0xFF).astype(np.uint8)
    for b in range(2):
        put_f16(w, b * 210 + 208, 0.05)
    out["q6k_pat_bytes"] = w
    out["q6k_pat_f32"] = quants.dequantize(w.reshape(2, 210), T.Q6_K).astype(np.float32).ravel()
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "kquant_decode.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
