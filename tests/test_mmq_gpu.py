"""Prefill MMQ (m > 8, Q4_K, tcgen05 kind::i8) vs the CPU restatement of infr-cpu's production path.

Two kernels sit behind Linear for m > 8.  The bit-identical one keeps the reference's arithmetic to the
last bit: exact int32 block sums (sd, sm) and one separately-rounded f32 expression per block,
accumulated in block order; its gate is bit identity of the f32 output, which implies bit-exact int32
accumulators.  The default, warp-specialised one has the same int32 block sums but fuses f32 roundings
and sums the min term over the whole row; the stated bar for f32 outputs is 1e-3 relative L2 and the
tests hold it to 1e-5 (the tensor core's f32 accumulation of the min term rounds toward zero, a bias of a few 1e-6).
"""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from fixtures import Q4K
from infr_b200 import synth

pytestmark = pytest.mark.gpu

WS_TOL = 1e-5  # f32 rounding noise; the bar for f32 outputs is 1e-3 relative L2


@pytest.fixture(scope="module")
def exact_backend():
    be = infr_b200.CudaBackend(device=0, mmq_kernel=1)
    yield be
    be.close()


@pytest.fixture(scope="module")
def ws_backend():
    """Every m > 8 Q4_K Linear on the warp-specialised GEMM, also the batches of a few dozen rows that the default
    context gives to the wide GEMV."""
    be = infr_b200.CudaBackend(device=0, mmq_kernel=2)
    yield be
    be.close()


SHAPES = [
    (9, 256, 8),          # one block, a sliver of a tile
    (64, 768, 128),       # exactly one tile, 3 blocks
    (70, 1024, 200),      # ragged in both tile dimensions
    (130, 2048, 300),
    (512, 4096, 1024),    # the prefill shape at reduced N
    (512, 4096, 14336),   # the prefill configuration itself: 112 row tiles x 8 token tiles, several tiles per persistent CTA
]


@pytest.mark.parametrize("m,in_f,out_f", SHAPES + [(200, 2560, 2100)])  # the last: several tiles per CTA wave
def test_mmq_ws_q4k_matches_production_cpu(ws_backend, oracle, m, in_f, out_f):
    w = synth.weight(Q4K, out_f, in_f, seed=m + in_f)
    x = synth.normal(6, (m, in_f))
    got = ws_backend.run_linear(Q4K, w, x, m, in_f, out_f)
    want = oracle.linear(Q4K, w, x, m, in_f, out_f)
    assert np.abs(want).max() > 1e-3
    assert fx.rel_l2(got, want) < WS_TOL
    # element-wise: the error of one output stays at rounding level of the largest output
    assert np.abs(got - want).max() <= 2e-5 * np.abs(want).max()


def test_mmq_ws_extreme_codes_do_not_overflow(ws_backend, oracle):
    m, in_f, out_f = 16, 512, 128
    blk = np.full(144, 0xFF, np.uint8)
    fx.put_f16(blk, 0, 0.01)
    fx.put_f16(blk, 2, 0.02)
    w = np.tile(blk, out_f * in_f // 256)
    x = np.where(np.arange(m * in_f).reshape(m, in_f) % 3 == 0, -1.0, 1.0).astype(np.float32)
    got = ws_backend.run_linear(Q4K, w, x, m, in_f, out_f)
    want = oracle.linear(Q4K, w, x, m, in_f, out_f)
    assert fx.rel_l2(got, want) < WS_TOL


def test_mmq_ws_large_activations(ws_backend, oracle):
    # activations in the thousands (outlier channels): the min-term operands stay inside tf32's f32 range
    m, in_f, out_f = 33, 1024, 256
    w = synth.weight(Q4K, out_f, in_f, seed=5)
    x = synth.normal(9, (m, in_f)) * 3000.0
    got = ws_backend.run_linear(Q4K, w, x, m, in_f, out_f)
    want = oracle.linear(Q4K, w, x, m, in_f, out_f)
    assert fx.rel_l2(got, want) < WS_TOL


@pytest.mark.parametrize("m,in_f,out_f", SHAPES)
def test_mmq_q4k_bit_identical_to_production_cpu(exact_backend, oracle, m, in_f, out_f):
    backend = exact_backend
    w = synth.weight(Q4K, out_f, in_f, seed=m + in_f)
    x = synth.normal(6, (m, in_f))
    got = backend.run_linear(Q4K, w, x, m, in_f, out_f)
    want = oracle.linear(Q4K, w, x, m, in_f, out_f)
    assert np.abs(want).max() > 1e-3
    assert fx.rel_l2(got, want) < 1e-3
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_mmq_extreme_codes_do_not_overflow(exact_backend, oracle):
    backend = exact_backend
    # all nibbles 15, all scales 63, activations pinned at +/-127: the largest |sd| the format allows
    m, in_f, out_f = 16, 512, 128
    blk = np.full(144, 0xFF, np.uint8)
    fx.put_f16(blk, 0, 0.01)
    fx.put_f16(blk, 2, 0.02)
    w = np.tile(blk, out_f * in_f // 256)
    x = np.where(np.arange(m * in_f).reshape(m, in_f) % 3 == 0, -1.0, 1.0).astype(np.float32)
    got = backend.run_linear(Q4K, w, x, m, in_f, out_f)
    want = oracle.linear(Q4K, w, x, m, in_f, out_f)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_mmq_matches_the_gemv_path_row_for_row(ws_backend):
    # a batch is m independent rows (crates/infr-cpu/src/kernels.rs:9297-9405): the GEMM and the
    # 8-row GEMV agree to f32 rounding order
    m, in_f, out_f = 24, 1024, 256
    w = synth.weight(Q4K, out_f, in_f, seed=77)
    x = synth.normal(78, (m, in_f))
    gemm = ws_backend.run_linear(Q4K, w, x, m, in_f, out_f)
    for r0 in range(0, m, 8):
        gemv = ws_backend.run_linear(Q4K, w, x[r0:r0 + 8], 8, in_f, out_f)
        assert fx.rel_l2(gemm[r0:r0 + 8], gemv) < 2e-5


@pytest.mark.parametrize("dt,m,in_f,out_f", [(Q4K, 32, 1024, 256), (Q4K, 19, 2048, 96), (infr_b200.Q6K, 32, 2048, 64), (infr_b200.Q6K, 27, 1024, 40),
                                             (infr_b200.Q2_0, 20, 1024, 48)])
def test_batches_of_a_few_dozen_rows(backend, oracle, dt, m, in_f, out_f):
    """Default context, 8 < m <= 32: Q4_K and Q6_K rows of whole 2048-element chunks take the wide GEMV, the other
    Q6_K shapes and Q2_0 are quantised once for all rows and walked 8 rows at a time."""
    w = synth.weight(dt, out_f, in_f, seed=91)
    x = synth.normal(92, (m, in_f))
    got = backend.run_linear(dt, w, x, m, in_f, out_f)
    want = oracle.linear(dt, w, x, m, in_f, out_f)
    assert fx.rel_l2(got, want) < WS_TOL
