"""The wide GEMV (gemv_wide.cu): Q4_K / Q6_K Linears over 9..32 rows per pass of the weights, the batch of a decode
step over a few dozen sequences.  A batch is m independent rows of the production dot products
(crates/infr-cpu/src/kernels.rs:2318 batch8, :2347-2688; :9297-9405 batch == single), so the gate is the production
CPU path row for row, and agreement with the 8-row GEMV walk."""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from infr_b200 import synth
from fixtures import Q4K, Q6K

pytestmark = pytest.mark.gpu

TOL = 1e-5  # f32 rounding noise; the bar for f32 outputs is 1e-3 relative L2


@pytest.fixture(scope="module")
def walk_backend():
    """Every batch walked through the GEMV 8 rows at a time."""
    be = infr_b200.CudaBackend(device=0, mmq_kernel=3)
    yield be
    be.close()


CASES = [
    # dtype, m, in_f, out_f
    (Q4K, 9, 256, 8),        # one super-block: one active warp, a sliver of a tile
    (Q4K, 16, 768, 40),      # three warps active, 2 row groups exactly
    (Q4K, 17, 2048, 100),    # a full K chunk, 3 row groups, ragged last tile
    (Q4K, 24, 2304, 333),    # two K chunks, the second with one block: partial results summed
    (Q4K, 25, 4096, 1024),
    (Q4K, 32, 4096, 4096),   # the attention projections of the 8B shape at batch 32
    (Q4K, 32, 14336, 4096),  # its FFN down: 7 K chunks
    (Q4K, 32, 4096, 14336),  # its FFN gate / up: many tiles per CTA
    (Q4K, 33, 1024, 96),     # one row more than a pass holds: the tensor-memory GEMM takes over
    (Q4K, 64, 2048, 520),
    (Q6K, 9, 2048, 8),
    (Q6K, 20, 2048, 100),
    (Q6K, 32, 4096, 1024),
    (Q6K, 32, 14336, 4096),  # the Q6_K FFN down of the Q4_K_M mix
    (Q6K, 31, 4096, 1000),   # odd row count of the matrix: the last tile is partial
    (Q6K, 80, 2048, 72),     # three passes (no Q6_K GEMM exists: every batch above 8 rows comes here)
]


@pytest.mark.parametrize("dt,m,in_f,out_f", CASES)
def test_wide_gemv_matches_production_cpu(backend, oracle, dt, m, in_f, out_f):
    w = synth.weight(dt, out_f, in_f, seed=in_f + out_f + m)
    x = synth.normal(m + 5, (m, in_f))
    got = backend.run_linear(dt, w, x, m, in_f, out_f)
    want = oracle.linear(dt, w, x, m, in_f, out_f)
    assert np.isfinite(got).all()
    assert fx.rel_l2(got, want) < TOL
    # row by row as well: one wrong row in a batch of 32 would hide in the norm of the whole
    for r in range(m):
        assert fx.rel_l2(got[r], want[r]) < 1e-4, r


@pytest.mark.parametrize("dt,m,in_f,out_f", [(Q4K, 29, 2304, 200), (Q6K, 29, 4096, 200)])
def test_wide_gemv_agrees_with_the_8_row_walk(backend, walk_backend, dt, m, in_f, out_f):
    w = synth.weight(dt, out_f, in_f, seed=5)
    x = synth.normal(6, (m, in_f))
    wide = backend.run_linear(dt, w, x, m, in_f, out_f)
    walk = walk_backend.run_linear(dt, w, x, m, in_f, out_f)
    assert fx.rel_l2(wide, walk) < 2e-5
    for r in range(m):
        assert fx.rel_l2(wide[r], walk[r]) < 1e-4, r


def test_extreme_codes_do_not_overflow(backend, oracle):
    """All weight nibbles 15 with the largest scales against saturated activations: the int32 sums stay exact."""
    m, in_f, out_f = 12, 1024, 32
    w = synth.weight(Q4K, out_f, in_f, seed=1).copy().reshape(out_f, -1, 144)
    w[:, :, 4:16] = 0xFF   # every 6-bit scale and min at 63
    w[:, :, 16:] = 0xFF    # every nibble 15
    w = w.reshape(-1)
    x = np.where(synth.normal(2, (m, in_f)) > 0, 1.0, -1.0).astype(np.float32) * 100.0
    got = backend.run_linear(Q4K, w, x, m, in_f, out_f)
    want = oracle.linear(Q4K, w, x, m, in_f, out_f)
    assert fx.rel_l2(got, want) < TOL


def test_run_twice_same_bits(backend):
    m, in_f, out_f = 32, 4096, 512
    w = synth.weight(Q4K, out_f, in_f, seed=3)
    x = synth.normal(4, (m, in_f))
    a = backend.run_linear(Q4K, w, x, m, in_f, out_f)
    b = backend.run_linear(Q4K, w, x, m, in_f, out_f)
    np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("dt", [Q4K, Q6K])
def test_two_weights_share_the_quantised_rows(backend, oracle, dt):
    m, in_f, o1, o2 = 32, 4096, 512, 136
    w1, w2 = synth.weight(dt, o1, in_f, seed=21), synth.weight(dt, o2, in_f, seed=22)
    x = synth.normal(23, (m, in_f))
    b1, b2 = backend.from_numpy(w1, infr_b200.USAGE_WEIGHTS), backend.from_numpy(w2, infr_b200.USAGE_WEIGHTS)
    xb, y1, y2 = backend.from_numpy(x), backend.alloc(m * o1 * 4), backend.alloc(m * o2 * 4)
    backend.linear_pair(dt, b1, y1, o1, b2, y2, o2, xb, m, in_f)
    for yb, w, o in ((y1, w1, o1), (y2, w2, o2)):
        got = backend.download(yb, np.float32).reshape(m, o)
        assert fx.rel_l2(got, oracle.linear(dt, w, x, m, in_f, o)) < TOL
    for b in (b1, b2, xb, y1, y2):
        b.close()


@pytest.mark.parametrize("dt,m,in_f,o1,o2", [(Q4K, 12, 2048, 200, 56), (Q4K, 32, 4096, 4096, 1024), (Q6K, 20, 4096, 136, 512),
                                             (Q4K, 9, 6144, 24, 1000)])
def test_pair_in_one_launch_has_the_bits_of_two_calls(backend, dt, m, in_f, o1, o2):
    """Two weights in one launch of the wide GEMV (and one launch that adds the K chunks of both): every tile and every
    chunk sum is computed as in a call of its own, so the results are the same bits - from f32 rows (linear_pair) and
    from pre-quantised rows (gemv_q8_pair)."""
    w1, w2 = synth.weight(dt, o1, in_f, seed=31), synth.weight(dt, o2, in_f, seed=32)
    x = synth.normal(33, (m, in_f))
    b1, b2 = backend.from_numpy(w1, infr_b200.USAGE_WEIGHTS), backend.from_numpy(w2, infr_b200.USAGE_WEIGHTS)
    xb = backend.from_numpy(x)
    ys = [backend.alloc(m * o * 4) for o in (o1, o2, o1, o2, o1, o2)]
    l0 = backend.launch_count()
    backend.linear_pair(dt, b1, ys[0], o1, b2, ys[1], o2, xb, m, in_f)
    n_pair = backend.launch_count() - l0
    backend.linear(dt, b1, xb, ys[2], m, in_f, o1)
    backend.linear(dt, b2, xb, ys[3], m, in_f, o2)
    n_two = backend.launch_count() - l0 - n_pair
    assert n_pair < n_two
    qs, d, s32, s16 = backend.alloc(m * in_f), backend.alloc(m * (in_f // 256) * 4), backend.alloc(m * (in_f // 32) * 4), backend.alloc(m * (in_f // 16) * 4)
    backend.quantize_q8(256, xb, m, in_f, qs, d, s32, s16)
    backend.gemv_q8_pair(dt, b1, ys[4], o1, b2, ys[5], o2, qs, d, s32, s16, m, in_f)
    got = [backend.download(y, np.float32) for y in ys]
    for k in (0, 1):
        np.testing.assert_array_equal(got[k].view(np.uint32), got[2 + k].view(np.uint32))
        np.testing.assert_array_equal(got[4 + k].view(np.uint32), got[2 + k].view(np.uint32))
    for b in [b1, b2, xb, qs, d, s32, s16] + ys:
        b.close()
