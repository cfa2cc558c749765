"""The non-matmul ops of a dense decode step, through the C ABI, against the CPU restatement of the reference's
CPU backend.  Integer / byte results are compared bit for bit; f32 results within the stated 1e-3 relative L2
(the assertions below are tighter: the two sides differ only in libm rounding and summation order)."""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from infr_b200 import synth

pytestmark = pytest.mark.gpu

TOL = 1e-3     # the bar for f32 outputs
TIGHT = 2e-5   # what these kernels are expected to meet


def _f16_cache(seed, rows, width):
    return synth.normal(seed, (rows, width)).astype(np.float16).view(np.uint16)


@pytest.mark.parametrize("rows,dim", [(1, 4096), (3, 4096), (2, 102), (5, 2048), (1, 8192)])
def test_rms_norm(backend, oracle, rows, dim):
    x = synth.normal(1, (rows, dim)) * 3.0
    w = 1.0 + 0.02 * synth.normal(2, (dim,))
    xb, wb, db = backend.from_numpy(x), backend.from_numpy(w), backend.alloc(rows * dim * 4)
    backend.rms_norm(xb, wb, db, rows, dim, 1e-5)
    got = backend.download(db, np.float32).reshape(rows, dim)
    assert fx.rel_l2(got, oracle.rms_norm(x, w, 1e-5)) < TIGHT < TOL


def test_add_rms_norm_in_place(backend, oracle):
    rows, dim = 4, 4096
    a, b = synth.normal(3, (rows, dim)), synth.normal(4, (rows, dim))
    w = 1.0 + 0.02 * synth.normal(5, (dim,))
    ab, bb, wb, nb = backend.from_numpy(a), backend.from_numpy(b), backend.from_numpy(w), backend.alloc(rows * dim * 4)
    backend.add_rms_norm(ab, bb, ab, wb, nb, rows, dim, 1e-5)
    h = oracle.add(a, b)
    np.testing.assert_array_equal(backend.download(ab, np.float32).reshape(rows, dim), h)  # Op::Add is exact
    assert fx.rel_l2(backend.download(nb, np.float32), oracle.rms_norm(h, w, 1e-5)) < TIGHT
    with pytest.raises(infr_b200.BackendError):
        backend.add_rms_norm(ab, bb, ab, wb, ab, rows, dim, 1e-5)  # the norm may not overwrite the sum


@pytest.mark.parametrize("neox", [False, True])
@pytest.mark.parametrize("n_head,head_dim,rope_dim", [(32, 128, 128), (4, 64, 32)])
def test_rope(backend, oracle, neox, n_head, head_dim, rope_dim):
    pos = np.array([0, 1, 77, 4096, 8191], np.int32)
    rows = pos.size
    x = synth.normal(6, (rows, n_head * head_dim))
    xb, pb, db = backend.from_numpy(x), backend.from_numpy(pos), backend.alloc(x.nbytes)
    backend.rope(xb, pb, db, rows, n_head, head_dim, rope_dim, 500000.0, neox)
    got = backend.download(db, np.float32).reshape(x.shape)
    want = oracle.rope(x, pos.astype(np.float32), n_head, head_dim, rope_dim, 500000.0, neox)
    # one ulp of difference in theta^(-2p/d) between the two libm's moves an angle by pos * 2^-24 radians
    assert fx.rel_l2(got, want) < 2e-4 < TOL
    # rotation keeps every pair's norm; dims beyond rope_dim pass through untouched
    g3 = got.reshape(rows, n_head, head_dim)
    np.testing.assert_array_equal(g3[:, :, rope_dim:], x.reshape(rows, n_head, head_dim)[:, :, rope_dim:])
    assert abs(np.linalg.norm(got) / np.linalg.norm(x) - 1) < 1e-6


def test_write_kv_is_bit_exact(backend, oracle):
    max_ctx, stride, rows, pos = 64, 1024, 3, 17
    src = synth.normal(7, (rows, stride)) * 4.0
    src[0, :4] = [65504.0, 1e-8, -0.0, 70000.0]  # max half, underflow, signed zero, overflow to inf
    cache = _f16_cache(8, max_ctx, stride).copy()
    cb = backend.from_numpy(cache)
    backend.write_kv(backend.from_numpy(src), cb, rows, stride, pos)
    want = cache.copy()
    oracle.write_kv_f16(src, want, rows, stride, pos)
    np.testing.assert_array_equal(backend.download(cb, np.uint16).reshape(max_ctx, stride), want)
    with pytest.raises(infr_b200.BackendError):
        backend.write_kv(backend.from_numpy(src), cb, rows, stride, max_ctx - 1)  # past the end of the cache


@pytest.mark.parametrize("n_head,n_kv,hd,pos,rows", [(8, 2, 128, 300, 1), (8, 2, 128, 127, 3), (4, 4, 64, 513, 2), (16, 2, 128, 5, 1),
                                                     (2, 1, 64, 0, 1), (32, 8, 128, 1100, 1)])
def test_attention(backend, oracle, n_head, n_kv, hd, pos, rows):
    ctx = pos + rows + 3
    kc, vc = _f16_cache(10, ctx, n_kv * hd), _f16_cache(11, ctx, n_kv * hd)
    q = synth.normal(12, (rows, n_head * hd))
    scale = 1.0 / np.sqrt(hd)
    qb, kb, vb, db = backend.from_numpy(q), backend.from_numpy(kc), backend.from_numpy(vc), backend.alloc(q.nbytes)
    backend.attention(qb, kb, vb, db, rows=rows, pos=pos, n_head=n_head, n_kv=n_kv, head_dim=hd, scale=scale)
    got = backend.download(db, np.float32).reshape(q.shape)
    want = oracle.attention(q, kc, vc, rows, n_head, n_kv, hd, scale, pos)
    assert fx.rel_l2(got, want) < TIGHT < TOL


@pytest.mark.parametrize("n_seq,n_head,n_kv,hd,pos", [(3, 8, 2, 128, 200),      # a single wave of CTAs: tiles fetched with cp.async
                                                      (16, 32, 8, 128, 1000),   # several waves: one bulk copy per row, partial last tile
                                                      (20, 8, 8, 64, 700)])     # the same with head_dim 64 (two warps per output group)
def test_attention_independent_sequences(backend, oracle, n_seq, n_head, n_kv, hd, pos):
    ctx = pos + 8
    stride = ctx * n_kv * hd
    kc, vc = _f16_cache(13, n_seq * ctx, n_kv * hd), _f16_cache(14, n_seq * ctx, n_kv * hd)
    q = synth.normal(15, (n_seq, n_head * hd))
    scale = 1.0 / np.sqrt(hd)
    qb, kb, vb, db = backend.from_numpy(q), backend.from_numpy(kc), backend.from_numpy(vc), backend.alloc(q.nbytes)
    backend.attention(qb, kb, vb, db, rows=1, pos=pos, n_head=n_head, n_kv=n_kv, head_dim=hd, scale=scale, n_seq=n_seq, seq_stride=stride)
    backend.sync()
    got = backend.download(db, np.float32).reshape(q.shape)
    for s in range(n_seq):
        want = oracle.attention(q[s], kc[s * ctx:(s + 1) * ctx], vc[s * ctx:(s + 1) * ctx], 1, n_head, n_kv, hd, scale, pos)
        assert fx.rel_l2(got[s], want) < TIGHT


def test_attention_rejects_unsupported_shapes(backend):
    b = backend.alloc(1 << 20)
    for kw in (dict(n_head=6, n_kv=2, head_dim=128), dict(n_head=8, n_kv=2, head_dim=96), dict(n_head=7, n_kv=2, head_dim=128)):
        with pytest.raises(infr_b200.BackendError):
            backend.attention(b, b, b, b, rows=1, pos=3, scale=1.0, **kw)


def test_rope_write_kv_matches_the_four_ops(backend, oracle):
    n_seq, n_head, n_kv, hd, pos, theta = 2, 8, 2, 128, 40, 500000.0
    ctx = 64
    stride = ctx * n_kv * hd
    q, k, v = synth.normal(16, (n_seq, n_head * hd)), synth.normal(17, (n_seq, n_kv * hd)), synth.normal(18, (n_seq, n_kv * hd))
    kc, vc = _f16_cache(19, n_seq * ctx, n_kv * hd).copy(), _f16_cache(20, n_seq * ctx, n_kv * hd).copy()
    positions = np.full(n_seq, pos, np.int32)
    qb, kcb, vcb = backend.from_numpy(q), backend.from_numpy(kc), backend.from_numpy(vc)
    backend.rope_write_kv(qb, backend.from_numpy(k), backend.from_numpy(v), backend.from_numpy(positions), kcb, vcb, rows=1, pos=pos,
                          n_head=n_head, n_kv=n_kv, head_dim=hd, theta=theta, n_seq=n_seq, seq_stride=stride)
    pf = positions.astype(np.float32)
    assert fx.rel_l2(backend.download(qb, np.float32), oracle.rope(q, pf, n_head, hd, hd, theta)) < TIGHT
    k_rot = oracle.rope(k, pf, n_kv, hd, hd, theta)
    want_k, want_v = kc.copy(), vc.copy()
    for s in range(n_seq):
        oracle.write_kv_f16(k_rot[s], want_k[s * ctx:(s + 1) * ctx], 1, n_kv * hd, pos)
        oracle.write_kv_f16(v[s], want_v[s * ctx:(s + 1) * ctx], 1, n_kv * hd, pos)
    got_k = backend.download(kcb, np.uint16).reshape(kc.shape)
    got_v = backend.download(vcb, np.uint16).reshape(vc.shape)
    np.testing.assert_array_equal(got_v, want_v)  # a plain cast: bit exact
    # the rotated k may differ from the CPU's by an f32 ulp before the cast: at most one f16 step, and rarely
    diff = np.abs(got_k.astype(np.int32) - want_k.astype(np.int32))
    assert diff.max() <= 1 and (diff != 0).mean() < 1e-3
    untouched = np.ones(kc.shape[0], bool)
    untouched[[pos, ctx + pos]] = False
    np.testing.assert_array_equal(got_k[untouched], kc[untouched])


def test_gated_act_and_add(backend, oracle):
    rows, nff = 3, 14336
    g, u = synth.normal(21, (rows, nff)) * 4.0, synth.normal(22, (rows, nff))
    gb, ub, db = backend.from_numpy(g), backend.from_numpy(u), backend.alloc(g.nbytes)
    backend.gated_act(gb, ub, db, rows, nff)
    assert fx.rel_l2(backend.download(db, np.float32), oracle.gated_act(g, u)) < TIGHT
    backend.add(gb, ub, db, rows * nff)
    np.testing.assert_array_equal(backend.download(db, np.float32), oracle.add(g, u).ravel())


def test_argmax_lowest_index_on_ties(backend, oracle):
    rows, n = 4, 128256
    x = synth.normal(23, (rows, n))
    x[1, 777] = x[1, 90000] = 50.0       # a tie: the lower index wins
    x[2, :] = -np.inf                    # nothing exceeds -inf: index 0
    x[3, 5] = np.nan
    x[3, n - 1] = 60.0
    xb, db = backend.from_numpy(x), backend.alloc(rows * 4)
    backend.argmax(xb, db, n, rows)
    got = backend.download(db, np.uint32)
    np.testing.assert_array_equal(got, oracle.argmax(x, n))
    assert got[1] == 777 and got[2] == 0 and got[3] == n - 1


def _q8_bufs(backend, rows, k):
    return backend.alloc(rows * k), backend.alloc(rows * k // 256 * 4), backend.alloc(rows * k // 32 * 4), backend.alloc(rows * k // 16 * 4)


def _q8_equal(backend, got, want):
    for g, w, dt in zip(got, want, (np.int8, np.uint32, np.int32, np.int32)):  # scales compared as bit patterns
        np.testing.assert_array_equal(backend.download(g, dt), backend.download(w, dt))


def test_producers_ending_in_the_quantiser_emit_the_quantisers_bits(backend, oracle):
    """add_rms_norm_q8 / gated_act_q8 / attention_q8 == the f32 op followed by quantize_q8, bit for bit; and the
    codes agree with the CPU quantiser applied to the CPU op's output wherever the f32 values agree."""
    rows, dim, nff = 3, 4096, 14336
    a, b = synth.normal(30, (rows, dim)), synth.normal(31, (rows, dim))
    w = (1.0 + 0.02 * synth.normal(32, (dim,))).astype(np.float32)
    ab, bb, wb = backend.from_numpy(a), backend.from_numpy(b), backend.from_numpy(w)
    sum1, sum2, nrm = backend.alloc(a.nbytes), backend.alloc(a.nbytes), backend.alloc(a.nbytes)
    want, got = _q8_bufs(backend, rows, dim), _q8_bufs(backend, rows, dim)
    backend.add_rms_norm(ab, bb, sum1, wb, nrm, rows, dim, 1e-5)
    backend.quantize_q8(256, nrm, rows, dim, *want)
    backend.add_rms_norm_q8(ab, bb, sum2, wb, rows, dim, 1e-5, *got)
    _q8_equal(backend, got, want)
    np.testing.assert_array_equal(backend.download(sum1, np.float32), backend.download(sum2, np.float32))
    qs_cpu, d_cpu, _, _ = oracle.quantize_q8(oracle.rms_norm(oracle.add(a, b), w, 1e-5))[:4]
    assert (backend.download(got[0], np.int8) != np.asarray(qs_cpu).ravel()).mean() < 1e-3  # f32 ulps can flip a rounding
    # without the residual
    backend.rms_norm(ab, wb, nrm, rows, dim, 1e-5)
    backend.quantize_q8(256, nrm, rows, dim, *want)
    backend.add_rms_norm_q8(ab, None, None, wb, rows, dim, 1e-5, *got)
    _q8_equal(backend, got, want)

    g, u = synth.normal(33, (rows, nff)) * 3.0, synth.normal(34, (rows, nff))
    gb, ub, act = backend.from_numpy(g), backend.from_numpy(u), backend.alloc(g.nbytes)
    want, got = _q8_bufs(backend, rows, nff), _q8_bufs(backend, rows, nff)
    backend.gated_act(gb, ub, act, rows, nff)
    backend.quantize_q8(256, act, rows, nff, *want)
    backend.gated_act_q8(gb, ub, rows, nff, *got)
    _q8_equal(backend, got, want)

    n_seq, n_head, n_kv, hd, pos = 2, 8, 2, 128, 333
    ctx = pos + 4
    kc, vc = _f16_cache(35, n_seq * ctx, n_kv * hd), _f16_cache(36, n_seq * ctx, n_kv * hd)
    q = synth.normal(37, (n_seq, n_head * hd))
    qb, kb, vb, ob = backend.from_numpy(q), backend.from_numpy(kc), backend.from_numpy(vc), backend.alloc(q.nbytes)
    kw = dict(rows=1, pos=pos, n_head=n_head, n_kv=n_kv, head_dim=hd, scale=0.088, n_seq=n_seq, seq_stride=ctx * n_kv * hd)
    want, got = _q8_bufs(backend, n_seq, n_head * hd), _q8_bufs(backend, n_seq, n_head * hd)
    backend.attention(qb, kb, vb, ob, **kw)
    backend.quantize_q8(256, ob, n_seq, n_head * hd, *want)
    backend.attention_q8(qb, kb, vb, *got, **kw)
    _q8_equal(backend, got, want)
    with pytest.raises(infr_b200.BackendError):
        backend.gated_act_q8(gb, ub, rows, 1000, *got)  # not whole 256-element blocks


def test_attention_with_a_position_per_sequence(backend, oracle):
    n_seq, n_head, n_kv, hd = 5, 8, 2, 128
    pos = np.array([300, 0, 127, 128, 1], np.int32)  # tile boundaries of 128 keys, an empty history
    ctx = int(pos.max()) + 4
    stride = ctx * n_kv * hd
    kc, vc = _f16_cache(21, n_seq * ctx, n_kv * hd), _f16_cache(22, n_seq * ctx, n_kv * hd)
    q = synth.normal(23, (n_seq, n_head * hd))
    scale = 1.0 / np.sqrt(hd)
    qb, kb, vb, db, pb = backend.from_numpy(q), backend.from_numpy(kc), backend.from_numpy(vc), backend.alloc(q.nbytes), backend.from_numpy(pos)
    backend.attention(qb, kb, vb, db, rows=1, pos=int(pos.max()), n_head=n_head, n_kv=n_kv, head_dim=hd, scale=scale, n_seq=n_seq, seq_stride=stride,
                      seq_pos=pb)
    got = backend.download(db, np.float32).reshape(q.shape)
    for s in range(n_seq):
        want = oracle.attention(q[s], kc[s * ctx:(s + 1) * ctx], vc[s * ctx:(s + 1) * ctx], 1, n_head, n_kv, hd, scale, int(pos[s]))
        assert fx.rel_l2(got[s], want) < TIGHT, s
    with pytest.raises(infr_b200.BackendError):  # the position array must cover every sequence
        backend.attention(qb, kb, vb, db, rows=1, pos=int(pos.max()), n_head=n_head, n_kv=n_kv, head_dim=hd, scale=scale, n_seq=n_seq,
                          seq_stride=stride, seq_pos=backend.from_numpy(pos[:2]))
