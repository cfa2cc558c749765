"""Pins the CPU restatement (oracle/) before anything is compared against it.

Every test cites the reference test it re-runs.  Literal known answers are used where the reference
has them; golden decode vectors come from tests/golden/kquant_decode.npz (independent `gguf`
implementation); everything else is the reference's own property test re-run on the restatement.
"""
import os

import numpy as np
import pytest

import fixtures as fx
from fixtures import Q2_0, Q4K, Q6K

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "kquant_decode.npz"))


# ---- geometry: crates/infr-core/src/decode_spec.rs:455-504 block_bytes_match_the_ggml_formulas ----
def test_block_bytes_match_the_ggml_formulas(oracle):
    QK_K = 256
    assert oracle.L.orc_block_bytes(Q4K) == 2 * 2 + 12 + QK_K // 2
    assert oracle.L.orc_block_bytes(Q6K) == QK_K // 2 + QK_K // 4 + QK_K // 16 + 2
    assert oracle.L.orc_block_bytes(Q2_0) == 2 + 64 // 4
    assert oracle.L.orc_block_elems(Q2_0) == 64


# ---- f16: half-crate semantics (exact widening, RNE narrowing) checked against numpy ----
def test_f16_roundtrip_all_bit_patterns(oracle):
    h = np.arange(65536, dtype=np.uint16)
    want = h.view(np.float16).astype(np.float32)
    got = np.array([oracle.f16_to_f32(int(v)) for v in h], np.float32)
    ok = (got.view(np.uint32) == want.view(np.uint32)) | (np.isnan(got) & np.isnan(want))
    assert ok.all()


def test_f32_to_f16_rne(oracle):
    rng = np.random.default_rng(0)
    vals = np.concatenate([
        rng.standard_normal(4000).astype(np.float32) * np.float32(10.0) ** rng.integers(-9, 6, 4000).astype(np.float32),
        np.array([0.0, -0.0, 65504.0, 65520.0, 65519.99, 1e-8, 6e-8, 5.96e-8, 2.98e-8, 3e-8, 0.05, 0.1, 0.375], np.float32),
    ])
    want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.f32_to_f16(float(v)) for v in vals], np.uint16)
    assert (got == want).all()


# ---- k4: crates/infr-gguf/src/dequant.rs:73-83 vs the packer in synth.quantize_q4k ----
def test_k4_unpacks_what_the_packer_packed(oracle):
    rng = np.random.default_rng(1)
    for _ in range(50):
        sc = rng.integers(0, 64, 8)
        mn = rng.integers(0, 64, 8)
        s = np.zeros(12, np.uint8)
        for k in range(4):
            s[k] = (sc[k] & 63) | (((sc[4 + k] >> 4) & 3) << 6)
            s[4 + k] = (mn[k] & 63) | (((mn[4 + k] >> 4) & 3) << 6)
            s[8 + k] = (sc[4 + k] & 0xF) | ((mn[4 + k] & 0xF) << 4)
        for j in range(8):
            assert oracle.k4(j, s) == (sc[j], mn[j])


# ---- literal known answer: crates/infr-gguf/src/dequant.rs:1406-1431 q2_0_single_block ----
def test_q2_0_single_block_known_answer(oracle):
    blk = np.zeros(18, np.uint8)
    fx.put_f16(blk, 0, 0.5)
    blk[2] = 0b11100100
    y = oracle.dequant(Q2_0, blk)
    assert y.shape == (64,)
    np.testing.assert_array_equal(y[:4], np.array([-0.5, 0.0, 0.5, 1.0], np.float32))
    np.testing.assert_array_equal(y[4:], np.full(60, -0.5, np.float32))


# ---- literal known answer: crates/infr-testkit/src/lib.rs:559-567 ----
def test_ref_linear_is_the_plain_dot_product(oracle):
    x = np.array([1, 2, 3, 4], np.float32)
    w = np.array([1, 10, 100, 1000], np.float32)
    got = oracle.ref_linear_f64(x, w, 2, 2, 2)
    np.testing.assert_array_equal(got.ravel(), np.array([21, 2100, 43, 4300], np.float32))


# ---- golden decode vectors from an independent implementation of the GGUF formats ----
@pytest.mark.parametrize("key,dt", [("q4k_lcg", Q4K), ("q6k_lcg", Q6K), ("q4k_pat", Q4K), ("q6k_pat", Q6K)])
def test_kquant_decode_matches_golden(oracle, key, dt):
    got = oracle.dequant(dt, GOLD[key + "_bytes"])
    want = GOLD[key + "_f32"]
    # both sides evaluate (d*sc)*q - (dmin*m) in f32; allow 1 ulp for a different association
    np.testing.assert_allclose(got, want, rtol=2e-7, atol=1e-9)
    assert np.abs(want).max() > 1e-3


# ---- crates/infr-core/src/decode_spec.rs:519-562 / testkit :529: scale slots are the scales ----
@pytest.mark.parametrize("dt", [Q4K, Q6K, Q2_0])
def test_doubling_d_doubles_magnitude(oracle, dt):
    w = fx.synth_weight(dt, 512, 0x77)
    base = oracle.dequant(dt, w)
    w2 = w.copy()
    be, bb = fx.BLOCK[dt]
    d, mn = fx.SYNTH_SCALES[dt]
    for b in range(512 // be):
        fx.put_f16(w2, b * bb + fx.D_SLOT[dt], 2 * d)
        if dt in fx.MIN_SLOT:
            fx.put_f16(w2, b * bb + fx.MIN_SLOT[dt], 2 * mn)
    np.testing.assert_allclose(oracle.dequant(dt, w2), 2 * base, rtol=2e-3, atol=1e-6)


# ---- quantisers: crates/infr-cpu/src/quant.rs:27-58, :97-117 ----
def test_quantize_q8_matches_numpy_restatement(oracle):
    x = fx.det_x(1024, 5)
    x[256:512] = 0.0  # an all-zero block: d = 0, id = 0, q = 0
    x[700] = -3.0
    qs, d, bs, bs16 = oracle.quantize_q8(x)
    for b in range(4):
        blk = x[b * 256:(b + 1) * 256]
        dd = np.float32(np.abs(blk).max()) / np.float32(127.0)
        assert d[b] == dd
        idv = np.float32(1.0) / dd if dd > 0 else np.float32(0)
        v = blk * idv
        want = np.clip(np.sign(v) * np.floor(np.abs(v) + np.float32(0.5)), -127, 127).astype(np.int8)
        np.testing.assert_array_equal(qs[b * 256:(b + 1) * 256], want)
    np.testing.assert_array_equal(bs16, qs.reshape(-1, 16).astype(np.int32).sum(1))
    np.testing.assert_array_equal(bs, qs.reshape(-1, 32).astype(np.int32).sum(1))
    assert d[1] == 0 and not qs[256:512].any()
    assert np.abs(qs).max() == 127


def test_quantize_q8_non_finite_elements_follow_rust_casts(oracle):
    """`(v * id).round().clamp(-127.0, 127.0) as i8` (quant.rs:38): f32::max skips a NaN when the block's amax is
    formed and the NaN's own code is 0 (`as i8` of a NaN); an infinite element makes d infinite and id 0, so every
    code of its block is 0; a block so small that 1 / (amax / 127) overflows gets +-127 for its non-zero elements."""
    x = np.linspace(-3.0, 3.0, 768, dtype=np.float32)
    x[5] = np.nan
    x[300] = np.inf
    x[512:768] *= np.float32(1e-38)
    x[512:600] *= np.float32(-1.0)
    x[600] = 0.0
    for qs, d in (oracle.quantize_q8(x)[:2], oracle.quantize_q8_32(x)[:2]):
        gran = x.size // d.size
        assert qs[5] == 0 and np.isfinite(d[0]) and d[0] == np.float32(np.nanmax(np.abs(x[:gran]))) / np.float32(127.0)
        assert np.isinf(d[300 // gran]) and not qs[300 // gran * gran:(300 // gran + 1) * gran].any()
        tiny = slice(512, 768)
        assert set(np.unique(qs[tiny])) <= {-127, 0, 127} and qs[600] == 0 and (qs[512:600] == -127).all() and (qs[640:768] == 127).all()


def test_quantize_q8_32_and_q8_1_share_codes(oracle):
    x = fx.det_x(704, 9) * np.float32(3.0)
    qs, d, bs = oracle.quantize_q8_32(x)
    np.testing.assert_array_equal(bs, qs.reshape(-1, 32).astype(np.int32).sum(1))
    qs1, dact, sact = oracle.quantize_q8_1(x)
    np.testing.assert_array_equal(qs, qs1)
    np.testing.assert_array_equal(dact, d.astype(np.float16).view(np.uint16))
    np.testing.assert_array_equal(sact, (d * bs.astype(np.float32)).astype(np.float16).view(np.uint16))


# ---- the 32-granular "Q8_1" GEMM tier of the reference's GPU backend
# (crates/infr-vulkan/shaders/native_gemm_mmq_q4k.comp:170-223, native_gemm_mmq_q6k.comp:151-219,
#  native_gemm_mmq_q2_0.comp:160-199): its integer block sums are the dequantised codes' dot products, and its f32
# result sits within quantisation distance of the production CPU tier and of the dequant reference.
@pytest.mark.parametrize("dt", [Q4K, Q6K, Q2_0])
def test_q8_1_gemm_tier_block_sums_and_distance_to_production(oracle, dt):
    import infr_b200.synth as synth
    m, in_f, out_f = 3, 512, 24
    w = synth.weight(dt, out_f, in_f, seed=40 + dt)
    x = np.stack([fx.det_x(in_f, 60 + r) * np.float32(1.0 + r) for r in range(m)])
    qa = np.empty((m, in_f), np.int8)
    dact = np.empty((m, in_f // 32), np.uint16)
    sact = np.empty((m, in_f // 32), np.uint16)
    for r in range(m):
        qa[r], dact[r], sact[r] = oracle.quantize_q8_1(x[r])
    got, qsum = oracle.mmq_q8_1(dt, w, qa, dact, sact, m, in_f, out_f, want_qsum=True)

    # Integer block sums: weight codes (no scale) against activation codes, exact.
    wq = np.asarray(w, np.uint8).reshape(out_f, -1)
    step = 16 if dt == Q6K else 32
    codes = np.empty((out_f, in_f), np.int64)
    for o in range(out_f):
        wz = wq[o].copy()
        be, bb = fx.BLOCK[dt]
        one = np.float16(1.0).view(np.uint16)
        for b in range(in_f // be):
            # d = 1, every sub-scale 1, min 0: dequant returns the bare codes (Q6_K: code-32, Q2_0: code-1).
            blk = wz[b * bb:(b + 1) * bb]
            if dt == Q4K:
                blk[0:2] = np.frombuffer(one.tobytes(), np.uint8); blk[2:4] = 0
                blk[4:8] = 1; blk[8:12] = 0; blk[12:16] = 1
            elif dt == Q6K:
                blk[192:208] = 1; blk[208:210] = np.frombuffer(one.tobytes(), np.uint8)
            else:
                blk[0:2] = np.frombuffer(one.tobytes(), np.uint8)
        codes[o] = np.rint(oracle.dequant(dt, wz)).astype(np.int64)
    want_qsum = np.einsum("okl,rkl->rok", codes.reshape(out_f, -1, step), qa.astype(np.int64).reshape(m, -1, step))
    np.testing.assert_array_equal(qsum, want_qsum)

    prod = oracle.linear(dt, w, x, m, in_f, out_f)
    ref = oracle.linear(dt, w, x, m, in_f, out_f, reference=True)
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    assert rel(got, ref) < 2e-2      # the reference's own production-vs-reference bar
    assert rel(got, prod) < 2e-2     # two quantisation granularities of the same activations
    assert rel(got, prod) > 0        # ... which are different computations


def _dequant_q8(q8, gran):
    qs, d = q8[0], q8[1]
    return (qs.reshape(-1, gran).astype(np.float32) * d[:, None]).ravel()


def _rel_err(got, want):
    return abs(float(got) - float(want)) / max(abs(float(want)), 1.0)


# ---- crates/infr-cpu/src/kernels.rs:6653-6666 q4k_dot_matches_dequant_reference ----
def test_q4k_dot_matches_dequant_reference(oracle):
    in_f = 768
    w = GOLD["q4k_lcg_bytes"]
    wref = oracle.dequant(Q4K, w)
    q8 = oracle.quantize_q8(fx.det_x(in_f, 2))
    got = oracle.vec_dot_q4k(w, q8, in_f)
    want = oracle.dot(wref, _dequant_q8(q8, 256))
    assert _rel_err(got, want) < 1e-3


# ---- crates/infr-cpu/src/kernels.rs:6669-6681 q6k_dot_matches_dequant_reference ----
def test_q6k_dot_matches_dequant_reference(oracle):
    in_f = 768
    w = GOLD["q6k_lcg_bytes"]
    wref = oracle.dequant(Q6K, w)
    q8 = oracle.quantize_q8(fx.det_x(in_f, 4))
    got = oracle.vec_dot_q6k(w, q8, in_f)
    want = oracle.dot(wref, _dequant_q8(q8, 256))
    assert _rel_err(got, want) < 1e-3


# ---- crates/infr-cpu/src/kernels.rs:7115-7160 q2_0_matches_dequant_reference ----
@pytest.mark.parametrize("in_f", [64, 256, 704])
def test_q2_0_matches_dequant_reference(oracle, in_f):
    nb = in_f // 64
    w = fx.det_bytes(nb * 18, 210)
    for k in range(nb):
        fx.put_f16(w, k * 18, 0.03)
    wref = oracle.dequant(Q2_0, w)
    assert np.any(wref[:64] != 0)
    for i in range(4):
        x = fx.det_x(in_f, 211 + i)
        q8 = oracle.quantize_q8_32(x)
        got = oracle.vec_dot_q2_0(w, q8, in_f)
        assert _rel_err(got, oracle.dot(wref, _dequant_q8(q8, 32))) < 1e-3
        assert _rel_err(got, oracle.dot(wref, x)) < 2e-2


# ---- integer accumulators equal an independent numpy integer evaluation ----
def test_block_accumulators_are_exact_integers(oracle):
    in_f = 1024
    x = fx.det_x(in_f, 77) * np.float32(4)
    q8 = oracle.quantize_q8(x)
    w4 = fx.synth_weight(Q4K, in_f, 0x31)
    _, sd, sm = oracle.vec_dot_q4k(w4, q8, in_f, want_acc=True)
    qa = q8[0].astype(np.int64)
    for b in range(in_f // 256):
        blk = w4[b * 144:(b + 1) * 144]
        qs = blk[16:]
        tsd = tsm = 0
        for s in range(8):
            sc, m = oracle.k4(s, blk[4:16])
            nib = (qs[(s // 2) * 32:(s // 2) * 32 + 32] >> (4 * (s & 1))) & 0xF
            a = qa[b * 256 + s * 32:b * 256 + s * 32 + 32]
            tsd += sc * int((nib.astype(np.int64) * a).sum())
            tsm += m * int(a.sum())
        assert (sd[b], sm[b]) == (tsd, tsm)
    w6 = fx.synth_weight(Q6K, in_f, 0x32)
    _, isum = oracle.vec_dot_q6k(w6, q8, in_f, want_acc=True)
    codes = np.rint(oracle.dequant(Q6K, _unit_scale_q6k(w6))).astype(np.int64)  # sc*(q-32) with d=1
    for b in range(in_f // 256):
        assert isum[b] == int((codes[b * 256:(b + 1) * 256] * qa[b * 256:(b + 1) * 256]).sum())


def _unit_scale_q6k(w):
    w = w.copy()
    for b in range(w.size // 210):
        fx.put_f16(w, b * 210 + 208, 1.0)
    return w


# ---- crates/infr-cpu/tests/decode_parity.rs:57-159: production 2e-2, reference 1e-5 ----
@pytest.mark.parametrize("dt", [Q4K, Q6K, Q2_0])
@pytest.mark.parametrize("m", [1, 2])
def test_linear_modes_against_the_f64_oracle(oracle, dt, m):
    in_f, out_f = 256, 8
    w, x = fx.case_inputs(dt, m, in_f, out_f, fx.weight_quant_case_seed(dt))
    want = oracle.ref_linear_f64(x, oracle.dequant(dt, w), m, in_f, out_f)
    ref_mag = np.abs(want).max()
    assert ref_mag > 1e-3
    prod = oracle.linear(dt, w, x, m, in_f, out_f)
    refm = oracle.linear(dt, w, x, m, in_f, out_f, reference=True)
    assert np.abs(prod - want).max() / ref_mag < 2e-2
    assert np.abs(refm - want).max() / ref_mag < 1e-5
    assert np.abs(prod - refm).max() / ref_mag < 2e-2


# ---- crates/infr-cpu/src/kernels.rs:9297-9405: a batch equals m single-row calls bit for bit ----
@pytest.mark.parametrize("dt", [Q4K, Q6K, Q2_0])
def test_batch_is_bit_identical_to_single_rows(oracle, dt):
    in_f, out_f, m = 512 if dt != Q2_0 else 704 - 704 % 64, 24, 5
    w = fx.synth_weight(dt, in_f * out_f, 0x99)
    x = np.stack([fx.det_x(in_f, 300 + r) for r in range(m)])
    batch = oracle.linear(dt, w, x, m, in_f, out_f)
    for r in range(m):
        one = oracle.linear(dt, w, x[r], 1, in_f, out_f)
        np.testing.assert_array_equal(batch[r].view(np.uint32), one[0].view(np.uint32))


# ---- dot: crates/infr-cpu/src/kernels.rs:6557-6573 (8 FMA lanes, in-order lane sum, FMA tail) ----
def test_dot_lane_structure(oracle):
    a = fx.det_x(37, 1)
    b = fx.det_x(37, 2)
    acc = np.zeros(8, np.float64)
    lanes = np.zeros(8, np.float32)
    for c in range(4):
        for j in range(8):
            lanes[j] = np.float32(np.float64(a[c * 8 + j]) * np.float64(b[c * 8 + j]) + np.float64(lanes[j]))
    s = np.float32(0)
    for j in range(8):
        s = np.float32(s + lanes[j])
    for i in range(32, 37):
        s = np.float32(np.float64(a[i]) * np.float64(b[i]) + np.float64(s))
    del acc
    assert oracle.dot(a, b) == s


# ---- MoE: crates/infr-llama/tests/seam_op_parity.rs:1224-1313 moe_ref (rows = 1, f32 reference) ----
def _moe_ref(o, x, router, gate, up, down, ne, n_expert, n_used, nff):
    logits = router.reshape(n_expert, ne).astype(np.float64) @ x.astype(np.float64)
    p = np.exp(logits - logits.max())
    p /= p.sum()
    order = sorted(range(n_expert), key=lambda e: -p[e])[:n_used]
    wsum = sum(p[e] for e in order)
    out = np.zeros(ne)
    gst, dst = nff * ne // 256 * 144, ne * nff // 256 * 144
    for e in order:
        g = o.dequant(Q4K, gate[e * gst:(e + 1) * gst]).reshape(nff, ne).astype(np.float64) @ x
        u = o.dequant(Q4K, up[e * gst:(e + 1) * gst]).reshape(nff, ne).astype(np.float64) @ x
        a = g / (1 + np.exp(-g)) * u
        y = o.dequant(Q4K, down[e * dst:(e + 1) * dst]).reshape(ne, nff).astype(np.float64) @ a
        out += p[e] / wsum * y
    return out, order


def test_moe_ffn_matches_f64_reference(oracle):
    from infr_b200 import synth

    ne, n_expert, n_used, nff = 256, 8, 2, 256
    router = synth.normal(11, (n_expert, ne), 1.0 / 16)
    gate = np.concatenate([synth.weight(Q4K, nff, ne, 100 + 3 * e) for e in range(n_expert)])
    up = np.concatenate([synth.weight(Q4K, nff, ne, 101 + 3 * e) for e in range(n_expert)])
    down = np.concatenate([synth.weight(Q4K, ne, nff, 102 + 3 * e) for e in range(n_expert)])
    x = synth.normal(12, (3, ne))
    kw = dict(rows=1, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=nff)
    for r in range(3):
        want, order = _moe_ref(oracle, x[r], router, gate, up, down, ne, n_expert, n_used, nff)
        got, ids, wts, _ = oracle.moe_ffn(x[r], router, gate, up, down, **kw)
        assert list(ids[0]) == order
        assert abs(wts.sum() - 1) < 1e-6
        assert fx.rel_l2(got, want) < 1e-5
    # rows >= 2 takes the int8 path (lib.rs:2359): within the int8 budget of the f64 reference,
    # and row-wise identical selection
    kw["rows"] = 3
    got, ids, _, _ = oracle.moe_ffn(x, router, gate, up, down, **kw)
    refm, ids_r, _, _ = oracle.moe_ffn(x, router, gate, up, down, reference=True, **kw)
    np.testing.assert_array_equal(ids, ids_r)
    for r in range(3):
        want, _ = _moe_ref(oracle, x[r], router, gate, up, down, ne, n_expert, n_used, nff)
        assert fx.rel_l2(refm[r], want) < 1e-5
        assert fx.rel_l2(got[r], want) < 2e-2
        assert fx.rel_l2(got[r], want) > 1e-6  # really went through int8 activations


def test_moe_top_k_ties_keep_the_lower_expert_id(oracle):
    from infr_b200 import synth

    ne, n_expert, n_used, nff = 256, 8, 3, 256
    router = np.zeros((n_expert, ne), np.float32)  # all logits equal -> all probs tie
    gate = np.concatenate([synth.weight(Q4K, nff, ne, 5) for _ in range(n_expert)])
    down = np.concatenate([synth.weight(Q4K, ne, nff, 6) for _ in range(n_expert)])
    x = synth.normal(3, (2, ne))
    _, ids, wts, _ = oracle.moe_ffn(x, router, gate, gate, down, rows=2, ne=ne, n_expert=n_expert,
                                    n_used=n_used, n_ff_exp=nff)
    np.testing.assert_array_equal(ids, np.array([[0, 1, 2], [0, 1, 2]], np.int32))
    np.testing.assert_allclose(wts, 1 / 3, rtol=1e-6)


# ---- the dense decode-step ops: the reference holds no literal vectors for them, so the restatement is pinned by
# ---- properties and by independent numpy / float64 evaluations of the same formulas
def test_rms_norm_properties(oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 512)).astype(np.float32) * 5
    w = (1 + 0.1 * rng.standard_normal(512)).astype(np.float32)
    y = oracle.rms_norm(x, w, 1e-5)
    want = x.astype(np.float64) / np.sqrt((x.astype(np.float64) ** 2).mean(1, keepdims=True) + 1e-5) * w
    assert fx.rel_l2(y, want) < 1e-6
    y1 = oracle.rms_norm(x, np.ones(512, np.float32), 0.0)
    np.testing.assert_allclose((y1.astype(np.float64) ** 2).mean(1), 1.0, rtol=1e-5)


@pytest.mark.parametrize("neox", [False, True])
def test_rope_is_a_rotation_by_relative_position(oracle, neox):
    rng = np.random.default_rng(2)
    nh, hd = 3, 64
    q = rng.standard_normal((1, nh * hd)).astype(np.float32)
    k = rng.standard_normal((1, nh * hd)).astype(np.float32)
    np.testing.assert_array_equal(oracle.rope(q, [0.0], nh, hd, hd, 10000.0, neox), q)  # position 0: identity
    # <rope(q, a), rope(k, b)> depends on a - b only, per head
    def dots(a, b):
        qa = oracle.rope(q, [a], nh, hd, hd, 10000.0, neox).reshape(nh, hd).astype(np.float64)
        kb = oracle.rope(k, [b], nh, hd, hd, 10000.0, neox).reshape(nh, hd).astype(np.float64)
        return (qa * kb).sum(1)
    np.testing.assert_allclose(dots(17.0, 5.0), dots(112.0, 100.0), atol=2e-4)
    # the first pair turns by exactly `pos` radians; a partial rope_dim leaves the tail alone
    r = oracle.rope(q, [2.0], nh, hd, 32, 10000.0, neox).reshape(nh, hd)
    i0, i1 = (0, 16) if neox else (0, 1)
    q3 = q.reshape(nh, hd)
    np.testing.assert_allclose(r[:, i0], q3[:, i0] * np.cos(2.0) - q3[:, i1] * np.sin(2.0), rtol=1e-5, atol=1e-6)
    np.testing.assert_array_equal(r[:, 32:], q3[:, 32:])


def test_write_kv_is_numpy_float16_rounding(oracle):
    rng = np.random.default_rng(3)
    src = (rng.standard_normal((2, 256)) * 10).astype(np.float32)
    src[0, :3] = [65504.0, 65520.0, 5.96e-8]
    cache = np.zeros((8, 256), np.uint16)
    oracle.write_kv_f16(src, cache, 2, 256, 3)
    with np.errstate(over="ignore"):
        np.testing.assert_array_equal(cache[3:5], src.astype(np.float16).view(np.uint16))
    assert not cache[:3].any() and not cache[5:].any()


def test_attention_against_float64_softmax(oracle):
    rng = np.random.default_rng(4)
    nh, nkv, hd, pos, rows = 4, 2, 64, 20, 2
    kc = rng.standard_normal((pos + rows, nkv * hd)).astype(np.float16)
    vc = rng.standard_normal((pos + rows, nkv * hd)).astype(np.float16)
    q = rng.standard_normal((rows, nh * hd)).astype(np.float32)
    got = oracle.attention(q, kc.view(np.uint16), vc.view(np.uint16), rows, nh, nkv, hd, 0.125, pos)
    want = np.empty_like(got, dtype=np.float64)
    for ti in range(rows):
        for h in range(nh):
            kv = h // (nh // nkv)
            K = kc[:pos + ti + 1, kv * hd:(kv + 1) * hd].astype(np.float64)
            V = vc[:pos + ti + 1, kv * hd:(kv + 1) * hd].astype(np.float64)
            sc = K @ q[ti, h * hd:(h + 1) * hd].astype(np.float64) * 0.125
            p = np.exp(sc - sc.max())
            want[ti, h * hd:(h + 1) * hd] = (p / p.sum()) @ V
    assert fx.rel_l2(got, want) < 1e-6
    # a single key: the output is that key's value row
    one = oracle.attention(q[:1], kc.view(np.uint16), vc.view(np.uint16), 1, nh, nkv, hd, 0.125, 0)
    np.testing.assert_array_equal(one.reshape(nh, hd)[0], vc[0, :hd].astype(np.float32))


def test_gated_act_add_argmax(oracle):
    rng = np.random.default_rng(5)
    g, u = rng.standard_normal(1000).astype(np.float32) * 3, rng.standard_normal(1000).astype(np.float32)
    want = g.astype(np.float64) / (1 + np.exp(-g.astype(np.float64))) * u
    assert fx.rel_l2(oracle.gated_act(g, u), want) < 1e-6
    np.testing.assert_array_equal(oracle.add(g, u), g + u)
    x = rng.standard_normal((3, 500)).astype(np.float32)
    x[1, 7] = x[1, 300] = 9.0
    x[2, :] = -np.inf
    np.testing.assert_array_equal(oracle.argmax(x, 500), [int(np.argmax(x[0])), 7, 0])
