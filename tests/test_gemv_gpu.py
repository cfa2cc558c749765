"""Decode GEMV (m <= 8) through the C ABI vs the CPU restatement of infr-cpu.

Gates: int32 block accumulators bit-exact; f32 outputs within 1e-3 relative L2 of the production
CPU path (the measured gap is ~1e-6: same integers, different order of the final f32 additions);
reference (f32-activation) mode within 1e-5 of max|oracle| like
crates/infr-cpu/tests/decode_parity.rs:93-102.
"""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from fixtures import Q2_0, Q4K, Q6K
from infr_b200 import synth

pytestmark = pytest.mark.gpu

TOL_REL_L2 = 1e-3       # the stated parity bar for final f32 outputs
TIGHT_REL_L2 = 2e-5     # what identical integer arithmetic actually delivers


def _gemv(backend, dt, w, x, m, in_f, out_f, act):
    wb = backend.from_numpy(w, infr_b200.USAGE_WEIGHTS)
    xb = backend.from_numpy(np.asarray(x, np.float32))
    yb = backend.alloc(m * out_f * 4)
    backend.gemv(dt, wb, xb, yb, m, in_f, out_f, act)
    y = backend.download(yb, np.float32).reshape(m, out_f)
    for b in (wb, xb, yb):
        b.close()
    return y


# ---- the reference's own seam cases: crates/infr-cpu/tests/decode_parity.rs (256x8, m=1 and 2) ----
@pytest.mark.parametrize("dt", [Q4K, Q6K, Q2_0])
@pytest.mark.parametrize("m", [1, 2])
def test_testkit_linear_cases(backend, oracle, dt, m):
    in_f, out_f = 256, 8
    w, x = fx.case_inputs(dt, m, in_f, out_f, fx.weight_quant_case_seed(dt))
    want64 = oracle.ref_linear_f64(x, oracle.dequant(dt, w), m, in_f, out_f)
    mag = np.abs(want64).max()
    assert mag > 1e-3
    prod = _gemv(backend, dt, w, x, m, in_f, out_f, infr_b200.ACT_INT8)
    refm = _gemv(backend, dt, w, x, m, in_f, out_f, infr_b200.ACT_F32)
    assert np.abs(prod - want64).max() / mag < 2e-2          # CPU_INT8_ACT_TOL
    assert np.abs(refm - want64).max() / mag < 1e-5          # reference-mode bound
    o_prod = oracle.linear(dt, w, x, m, in_f, out_f)
    assert fx.rel_l2(prod, o_prod) < TIGHT_REL_L2
    # through the graph seam (compile / bind / execute / download) the result is the same
    seam = backend.run_linear(dt, w, x, m, in_f, out_f)
    np.testing.assert_array_equal(seam, prod)


SHAPES = [
    (Q4K, 768, 40),      # 3 super-blocks: a partial 4-block warp step
    (Q4K, 2048, 768),    # MoE expert gate/up
    (Q4K, 4096, 4096),   # the Q4_K 4096x4096 matvec configuration
    (Q4K, 1024, 6408),   # 401 row tiles (the last one partial): the 8-warps-per-tile configuration
    (Q4K, 14336, 1000),  # long rows: 56 super-blocks split over the warps of a tile
    (Q6K, 768, 24),
    (Q6K, 4096, 14336),  # decode sweep: W 14336 x 4096 in Q6_K (matrix-unit kernel: 16 blocks, odd ones off a word boundary)
    (Q6K, 2048, 100),    # 8 blocks over 16 warps (half of them idle), partial last 16-row tile
    (Q6K, 14336, 520),   # 56 blocks per row
    (Q6K, 4096, 4000),   # eight warps per tile
    (Q2_0, 704, 16),     # 11 blocks: not a multiple of 8 blocks nor of 256 elements
    (Q2_0, 14336, 4096), # decode sweep: ternary W 4096 x 14336 (matrix-unit kernel, 28 chunks over 4 warps)
    (Q2_0, 512, 40),     # one 512-element chunk, partial last 16-row tile (16 warps, most of them idle)
    (Q2_0, 2048, 6408),  # many tiles: four warps per tile, one chunk each
    (Q2_0, 4096, 2500),  # eight warps per tile, partial last tile
]


def _weight(dt, out_f, in_f, seed):
    return synth.weight(dt, out_f, in_f, seed)


@pytest.mark.parametrize("dt,in_f,out_f", SHAPES)
@pytest.mark.parametrize("m", [1, 4, 8])
def test_int8_gemv_matches_production_cpu(backend, oracle, dt, in_f, out_f, m):
    w = _weight(dt, out_f, in_f, seed=in_f + out_f + dt)
    x = synth.normal(4 + m, (m, in_f))
    got = _gemv(backend, dt, w, x, m, in_f, out_f, infr_b200.ACT_INT8)
    want = oracle.linear(dt, w, x, m, in_f, out_f)
    rel = fx.rel_l2(got, want)
    assert rel < TOL_REL_L2 and rel < TIGHT_REL_L2, rel
    for r in range(m):
        assert int(np.argmax(got[r])) == int(np.argmax(want[r]))


@pytest.mark.parametrize("m", [2, 3, 5, 6, 7])
def test_every_batch_width(backend, oracle, m):
    for dt, in_f, out_f in [(Q4K, 1024, 64), (Q6K, 512, 48), (Q2_0, 320, 40)]:
        w = synth.weight(dt, out_f, in_f, seed=m)
        x = synth.normal(50 + m, (m, in_f))
        got = _gemv(backend, dt, w, x, m, in_f, out_f, infr_b200.ACT_INT8)
        assert fx.rel_l2(got, oracle.linear(dt, w, x, m, in_f, out_f)) < TIGHT_REL_L2


@pytest.mark.parametrize("dt,in_f,out_f", SHAPES)
def test_block_accumulators_bit_exact(backend, oracle, dt, in_f, out_f):
    out_f = min(out_f, 512)
    w = _weight(dt, out_f, in_f, seed=7 * in_f + dt)
    x = synth.normal(9, (1, in_f)) * np.float32(3.0)
    per = {Q4K: in_f // 256 * 2, Q6K: in_f // 256, Q2_0: in_f // 32}[dt]
    wb = backend.from_numpy(w, infr_b200.USAGE_WEIGHTS)
    xb = backend.from_numpy(x)
    ab = backend.alloc(out_f * per * 4)
    backend.gemv_block_acc(dt, wb, xb, ab, in_f, out_f)
    got = backend.download(ab, np.int32).reshape(out_f, per)
    bpr = synth.row_bytes(dt, in_f)
    q8 = oracle.quantize_q8(x[0]) if dt != Q2_0 else oracle.quantize_q8_32(x[0])
    for o in range(out_f):
        row = w[o * bpr:(o + 1) * bpr]
        if dt == Q4K:
            _, sd, sm = oracle.vec_dot_q4k(row, q8, in_f, want_acc=True)
            want = np.stack([sd, sm], 1).ravel()
        elif dt == Q6K:
            _, want = oracle.vec_dot_q6k(row, q8, in_f, want_acc=True)
        else:
            _, want = oracle.vec_dot_q2_0(row, q8, in_f, want_acc=True)
        np.testing.assert_array_equal(got[o], want)


@pytest.mark.parametrize("dt,in_f,out_f", SHAPES)
@pytest.mark.parametrize("m", [1, 3])
def test_f32_gemv_matches_reference_mode(backend, oracle, dt, in_f, out_f, m):
    out_f = min(out_f, 2048)
    w = _weight(dt, out_f, in_f, seed=11 * in_f + dt)
    x = synth.normal(13 + m, (m, in_f))
    got = _gemv(backend, dt, w, x, m, in_f, out_f, infr_b200.ACT_F32)
    want = oracle.linear(dt, w, x, m, in_f, out_f, reference=True)
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-5
    assert fx.rel_l2(got, want) < 1e-5
    # and the two CPU modes differ by the int8 activation error, far more than either GPU gap
    prod = oracle.linear(dt, w, x, m, in_f, out_f)
    assert fx.rel_l2(prod, want) > 1e-4


def test_determinism_run_twice(backend):
    in_f, out_f = 4096, 1024
    for dt in (Q4K, Q6K, Q2_0):
        w = synth.weight(dt, out_f, in_f if dt != Q2_0 else 4096, seed=3)
        x = synth.normal(5, (8, in_f))
        a = _gemv(backend, dt, w, x, 8, in_f, out_f, infr_b200.ACT_INT8)
        b = _gemv(backend, dt, w, x, 8, in_f, out_f, infr_b200.ACT_INT8)
        np.testing.assert_array_equal(a.view(np.uint32), b.view(np.uint32))


def test_w_off_selects_rows_of_a_fused_weight(backend, oracle):
    # fused QKV: three projections stacked in one weight, addressed by w_off (graph.rs:186-190)
    in_f, rows = 512, [64, 16, 16]
    w = synth.weight(Q4K, sum(rows), in_f, seed=21)
    x = synth.normal(22, (1, in_f))
    bpr = synth.row_bytes(Q4K, in_f)
    r0 = 0
    for n in rows:
        got = backend.run_linear(Q4K, w, x, 1, in_f, n, w_off=r0 * in_f, total_rows=sum(rows))
        want = oracle.linear(Q4K, w[r0 * bpr:(r0 + n) * bpr], x, 1, in_f, n)
        assert fx.rel_l2(got, want) < TIGHT_REL_L2
        r0 += n


def test_wide_batch_falls_through_linear(backend, oracle):
    in_f, out_f, m = 512, 96, 19
    w = synth.weight(Q6K, out_f, in_f, seed=31)
    x = synth.normal(32, (m, in_f))
    got = backend.run_linear(Q6K, w, x, m, in_f, out_f)
    assert fx.rel_l2(got, oracle.linear(Q6K, w, x, m, in_f, out_f)) < TIGHT_REL_L2


def test_errors_are_returned_not_raised_as_faults(backend):
    g = infr_b200.Graph()
    xid = g.input(256)
    wid = g.weight(256 * 8, Q4K)
    dst = g.output(8)
    g.linear(xid, wid, dst, 1, 256, 8)
    plan = backend.compile(g)
    xb = backend.alloc(1024)
    with pytest.raises(infr_b200.BackendError) as ei:      # unbound weight handle
        backend.execute(plan, {xid: xb})
    assert ei.value.code == infr_b200.E_INVALID and "unbound" in str(ei.value)
    small = backend.alloc(100)
    ob = backend.alloc(32)
    with pytest.raises(infr_b200.BackendError) as ei:      # weight buffer too small
        backend.execute(plan, {xid: xb, wid: small, dst: ob})
    assert ei.value.code == infr_b200.E_INVALID
    g2 = infr_b200.Graph()
    a = g2.input(100)
    b = g2.weight(100 * 8, Q4K)
    c = g2.output(8)
    g2.linear(a, b, c, 1, 100, 8)
    # 100 is not a whole number of 256-element blocks
    wbuf = backend.alloc(4096)
    p2 = backend.compile(g2)
    with pytest.raises(infr_b200.BackendError):
        backend.execute(p2, {a: xb, b: wbuf, c: ob})
    g3 = infr_b200.Graph()
    a = g3.input(256)
    b = g3.weight(256 * 8, infr_b200.F32 + 5)   # Q4_0: a dtype this backend does not run
    c = g3.output(8)
    g3.linear(a, b, c, 1, 256, 8)
    with pytest.raises(infr_b200.BackendError) as ei:
        backend.compile(g3)
    assert ei.value.code == infr_b200.E_UNSUPPORTED
    with pytest.raises(infr_b200.BackendError):             # upload larger than the buffer
        backend.upload(small, np.zeros(200, np.uint8))
    caps = backend.capabilities()
    assert caps.name == "cuda-sm100a" and caps.i8_dot and not caps.unified_memory and caps.sm_count > 0


@pytest.mark.parametrize("dt,in_f,out1,out2,m", [(Q4K, 1024, 320, 96, 1), (Q4K, 1024, 333, 40, 5), (Q4K, 4096, 4096, 1024, 1),
                                                 (Q4K, 2048, 24, 7000, 8), (Q6K, 2048, 64, 48, 2)])
def test_two_weights_against_the_same_rows_in_one_call(backend, oracle, dt, in_f, out1, out2, m):
    """infr_cuda_gemv_q8_pair (q and k, gate and up of a decode step): both results as from two separate calls (the
    integer block sums are the same; one launch may split K over a different number of warps, which reorders the f32
    additions) and within the parity bar of the CPU."""
    w1, w2 = synth.weight(dt, out1, in_f, seed=11), synth.weight(dt, out2, in_f, seed=12)
    x = synth.normal(13, (m, in_f))
    b1, b2 = backend.from_numpy(w1, infr_b200.USAGE_WEIGHTS), backend.from_numpy(w2, infr_b200.USAGE_WEIGHTS)
    xb = backend.from_numpy(x)
    qs, d, s32, s16 = backend.alloc(m * in_f), backend.alloc(m * (in_f // 256) * 4), backend.alloc(m * (in_f // 32) * 4), backend.alloc(m * (in_f // 16) * 4)
    backend.quantize_q8(256, xb, m, in_f, qs, d, s32, s16)
    y1, y2, z1, z2 = (backend.alloc(m * o * 4) for o in (out1, out2, out1, out2))
    backend.gemv_q8_pair(dt, b1, y1, out1, b2, y2, out2, qs, d, s32, s16, m, in_f)
    backend.gemv_q8(dt, b1, qs, d, s32, s16, z1, m, in_f, out1)
    backend.gemv_q8(dt, b2, qs, d, s32, s16, z2, m, in_f, out2)
    for got_b, ref_b, w, o in ((y1, z1, w1, out1), (y2, z2, w2, out2)):
        got, ref = backend.download(got_b, np.float32).reshape(m, o), backend.download(ref_b, np.float32).reshape(m, o)
        assert fx.rel_l2(got, ref) < TIGHT_REL_L2
        assert fx.rel_l2(got, oracle.linear(dt, w, x, m, in_f, o)) < TIGHT_REL_L2
    for b in (b1, b2, xb, qs, d, s32, s16, y1, y2, z1, z2):
        b.close()
