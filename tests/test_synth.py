"""Host-side block packers: what they emit must decode (through the CPU checker) to what went in."""
import numpy as np

from infr_b200 import synth
from fixtures import Q2_0, Q4K, Q6K


def test_row_bytes():
    assert synth.row_bytes(Q4K, 4096) == 2304
    assert synth.row_bytes(Q6K, 4096) == 3360
    assert synth.row_bytes(Q2_0, 14336) == 4032


def test_q4k_pack_round_trip(oracle):
    w = synth.normal(0, (8, 512), 0.02)
    raw = synth.quantize_q4k(w)
    assert raw.size == 8 * 2 * 144
    back = oracle.dequant(Q4K, raw).reshape(8, 512)
    err = np.abs(back - w).max()
    assert err < 0.02 * 6 / 15  # within one quantisation step of the widest sub-block
    assert np.linalg.norm(back - w) / np.linalg.norm(w) < 0.08


def test_q6k_pack_round_trip(oracle):
    w = synth.normal(2, (8, 512), 0.02)
    raw = synth.quantize_q6k(w)
    assert raw.size == 8 * 2 * 210
    back = oracle.dequant(Q6K, raw).reshape(8, 512)
    assert np.linalg.norm(back - w) / np.linalg.norm(w) < 0.03


def test_q2_0_pack_round_trip(oracle):
    raw = synth.weight(Q2_0, 4, 256, seed=3)
    back = oracle.dequant(Q2_0, raw).reshape(4, 4, 64)
    d = raw.reshape(-1, 18)[:, :2].copy().view(np.float16).astype(np.float32).reshape(4, 4, 1)
    tern = np.rint(back / d)
    assert set(np.unique(tern)) <= {-1.0, 0.0, 1.0}
    frac0 = (tern == 0).mean()
    assert 0.35 < frac0 < 0.65


def test_seeds_are_reproducible():
    a = synth.weight(Q4K, 16, 256, seed=5)
    b = synth.weight(Q4K, 16, 256, seed=5)
    c = synth.weight(Q4K, 16, 256, seed=6)
    assert (a == b).all() and (a != c).any()
