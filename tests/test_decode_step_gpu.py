"""A whole decode step (small Llama-shaped model, two sequences) through the C ABI against the same op sequence
evaluated with the CPU restatement: same argmax, logits within the stated 1e-3 relative L2, KV rows written."""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from infr_b200 import Q4K, Q6K, synth
from infr_b200.decode import DecodeStep, LlamaShape

pytestmark = pytest.mark.gpu

SHAPE = LlamaShape(n_layer=2, hidden=512, n_head=4, n_kv=2, head_dim=128, ffn=1024, vocab=1000)
N_SEQ, MAX_CTX, POS = 2, 48, 37


def _model(seed0=1000):
    s = SHAPE
    layers = []
    for li in range(s.n_layer):
        L = {}
        for t, (name, dt, o, i) in enumerate(s.linears()):
            L[name] = (dt, synth.weight(dt, o, i, seed=seed0 + li * 16 + t), o, i)
        L["attn_norm"] = (1.0 + 0.02 * synth.normal(seed0 + li * 16 + 8, (s.hidden,))).astype(np.float32)
        L["ffn_norm"] = (1.0 + 0.02 * synth.normal(seed0 + li * 16 + 9, (s.hidden,))).astype(np.float32)
        layers.append(L)
    out_norm = (1.0 + 0.02 * synth.normal(seed0 + 900, (s.hidden,))).astype(np.float32)
    head = synth.weight(Q4K, s.vocab, s.hidden, seed=seed0 + 901)
    kc = [synth.normal(9 + 2 * li, (N_SEQ * MAX_CTX, s.kv_dim)).astype(np.float16).view(np.uint16) for li in range(s.n_layer)]
    vc = [synth.normal(10 + 2 * li, (N_SEQ * MAX_CTX, s.kv_dim)).astype(np.float16).view(np.uint16) for li in range(s.n_layer)]
    return layers, out_norm, head, kc, vc


def _oracle_step(o, layers, out_norm, head, kc, vc, hidden):
    """The reference's op order on the CPU restatement; kc / vc are modified in place."""
    s, b = SHAPE, N_SEQ
    scale = 1.0 / np.sqrt(s.head_dim)
    pos = np.full(b, POS, np.float32)
    lin = lambda w, x: o.linear(w[0], w[1], x, b, w[3], w[2])
    hidden = hidden.copy()
    for li, L in enumerate(layers):
        hn = o.rms_norm(hidden, L["attn_norm"], s.eps)
        q, k, v = lin(L["wq"], hn), lin(L["wk"], hn), lin(L["wv"], hn)
        k16 = o.rope(k, pos, s.n_kv, s.head_dim, s.head_dim, s.theta)
        q = o.rope(q, pos, s.n_head, s.head_dim, s.head_dim, s.theta)
        attn = np.empty((b, s.q_dim), np.float32)
        for sq in range(b):
            ks, vs = kc[li][sq * MAX_CTX:(sq + 1) * MAX_CTX], vc[li][sq * MAX_CTX:(sq + 1) * MAX_CTX]
            o.write_kv_f16(k16[sq], ks, 1, s.kv_dim, POS)
            o.write_kv_f16(v[sq], vs, 1, s.kv_dim, POS)
            attn[sq] = o.attention(q[sq], ks, vs, 1, s.n_head, s.n_kv, s.head_dim, scale, POS)
        hidden = o.add(hidden, lin(L["wo"], attn))
        hn = o.rms_norm(hidden, L["ffn_norm"], s.eps)
        act = o.gated_act(lin(L["gate"], hn), lin(L["up"], hn))
        hidden = o.add(hidden, lin(L["down"], act))
    hn = o.rms_norm(hidden, out_norm, s.eps)
    logits = o.linear(Q4K, head, hn, b, s.hidden, s.vocab)
    return logits, o.argmax(logits, s.vocab)


@pytest.mark.parametrize("fused,q8_fused", [(False, False), (True, False), (True, True)], ids=["op-by-op", "fused", "fused-int8"])
def test_decode_step_matches_the_cpu_op_sequence(backend, oracle, fused, q8_fused):
    s = SHAPE
    layers, out_norm, head, kc, vc = _model()
    hidden = synth.normal(77, (N_SEQ, s.hidden))
    dev_layers = []
    for L in layers:
        d = {name: backend.from_numpy(L[name][1], infr_b200.USAGE_WEIGHTS) for name, *_ in s.linears()}
        d["attn_norm"], d["ffn_norm"] = backend.from_numpy(L["attn_norm"]), backend.from_numpy(L["ffn_norm"])
        dev_layers.append(d)
    kcb, vcb = [backend.from_numpy(c) for c in kc], [backend.from_numpy(c) for c in vc]
    step = DecodeStep(backend, s, N_SEQ, MAX_CTX, dev_layers, backend.from_numpy(out_norm), backend.from_numpy(head, infr_b200.USAGE_WEIGHTS),
                      Q4K, kcb, vcb)
    step.set_inputs(hidden, POS)
    n_ops = step.run(POS, fused=fused, q8_fused=q8_fused)
    assert n_ops > 0
    got_logits = backend.download(step.logits, np.float32).reshape(N_SEQ, s.vocab)
    got_tok = backend.download(step.tok, np.uint32)

    want_kc, want_vc = [c.copy() for c in kc], [c.copy() for c in vc]
    want_logits, want_tok = _oracle_step(oracle, layers, out_norm, head, want_kc, want_vc, hidden)
    err = fx.rel_l2(got_logits, want_logits)
    assert err < 1e-3, err
    np.testing.assert_array_equal(got_tok, want_tok)
    print(f"decode step fused={fused} int8-producers={q8_fused}: logits rel-L2 {err:.2e}, max-abs-diff {np.abs(got_logits - want_logits).max():.3e}")
    # the new V rows are plain casts of a Linear output: compare as values (the Linear differs in f32 rounding)
    for li in range(s.n_layer):
        g = backend.download(vcb[li], np.uint16).reshape(vc[li].shape)
        rows = [POS, MAX_CTX + POS]
        assert fx.rel_l2(g[rows].view(np.float16).astype(np.float32), want_vc[li][rows].view(np.float16).astype(np.float32)) < 2e-3
        keep = np.ones(g.shape[0], bool)
        keep[rows] = False
        np.testing.assert_array_equal(g[keep], vc[li][keep])


def test_a_dozen_sequences_keep_int8_activations_between_ops(backend):
    """9..32 sequences with every Linear on the wide GEMV: the step runs its int8-producer form (RMSNorm, attention
    merge and SiLU gate end in the quantiser, Linears take the codes) and gives what the op-by-op form gives."""
    s = LlamaShape(n_layer=2, hidden=2048, n_head=16, n_kv=4, head_dim=128, ffn=2048, vocab=512)
    b, ctx, pos = 12, 24, 9
    dev_layers = []
    for li in range(s.n_layer):
        d = {name: backend.from_numpy(synth.weight(dt, o, i, seed=2000 + 16 * li + t), infr_b200.USAGE_WEIGHTS)
             for t, (name, dt, o, i) in enumerate(s.linears())}
        d["attn_norm"] = backend.from_numpy((1.0 + 0.02 * synth.normal(2100 + li, (s.hidden,))).astype(np.float32))
        d["ffn_norm"] = backend.from_numpy((1.0 + 0.02 * synth.normal(2200 + li, (s.hidden,))).astype(np.float32))
        dev_layers.append(d)
    out_norm = backend.from_numpy((1.0 + 0.02 * synth.normal(2300, (s.hidden,))).astype(np.float32))
    head = backend.from_numpy(synth.weight(Q6K, s.vocab, s.hidden, seed=2301), infr_b200.USAGE_WEIGHTS)
    kc = [synth.normal(50 + li, (b * ctx, s.kv_dim)).astype(np.float16).view(np.uint16) for li in range(s.n_layer)]
    vc = [synth.normal(60 + li, (b * ctx, s.kv_dim)).astype(np.float16).view(np.uint16) for li in range(s.n_layer)]
    hidden = synth.normal(70, (b, s.hidden))
    outs = []
    for fused, q8 in ((False, False), (True, None)):
        step = DecodeStep(backend, s, b, ctx, dev_layers, out_norm, head, Q6K, [backend.from_numpy(c) for c in kc], [backend.from_numpy(c) for c in vc])
        assert step._wide_ok()
        step.set_inputs(hidden, pos)
        l0 = backend.launch_count()
        step.run(pos, fused=fused, q8_fused=q8)
        outs.append((backend.download(step.logits, np.float32).reshape(b, s.vocab), backend.download(step.tok, np.uint32), backend.launch_count() - l0))
    (ref_logits, ref_tok, ref_launches), (got_logits, got_tok, got_launches) = outs
    assert np.isfinite(got_logits).all()
    assert fx.rel_l2(got_logits, ref_logits) < 1e-5
    np.testing.assert_array_equal(got_tok, ref_tok)
    assert got_launches < ref_launches


def test_sequences_at_positions_of_their_own(backend, oracle):
    """A continuously served batch: every sequence has its own length.  Each sequence's logits are those of the same
    sequence run alone at its position (the CPU op sequence per sequence), in the op-by-op, fused and int8-producer forms."""
    s = SHAPE
    layers, out_norm, head, kc, vc = _model(seed0=3000)
    b, positions = N_SEQ, np.array([5, 31], np.int32)
    hidden = synth.normal(78, (b, s.hidden))
    dev_layers = []
    for L in layers:
        d = {name: backend.from_numpy(L[name][1], infr_b200.USAGE_WEIGHTS) for name, *_ in s.linears()}
        d["attn_norm"], d["ffn_norm"] = backend.from_numpy(L["attn_norm"]), backend.from_numpy(L["ffn_norm"])
        dev_layers.append(d)
    on, hd = backend.from_numpy(out_norm), backend.from_numpy(head, infr_b200.USAGE_WEIGHTS)
    # the CPU: one sequence at a time at its own position
    want = np.empty((b, s.vocab), np.float32)
    scale = 1.0 / np.sqrt(s.head_dim)
    for sq in range(b):
        pos = int(positions[sq])
        lin = lambda w, x: oracle.linear(w[0], w[1], x, 1, w[3], w[2])
        h = hidden[sq:sq + 1].copy()
        for li, L in enumerate(layers):
            hn = oracle.rms_norm(h, L["attn_norm"], s.eps)
            q, k, v = lin(L["wq"], hn), lin(L["wk"], hn), lin(L["wv"], hn)
            pf = np.full(1, pos, np.float32)
            k16 = oracle.rope(k, pf, s.n_kv, s.head_dim, s.head_dim, s.theta)
            q = oracle.rope(q, pf, s.n_head, s.head_dim, s.head_dim, s.theta)
            ks, vs = kc[li][sq * MAX_CTX:(sq + 1) * MAX_CTX].copy(), vc[li][sq * MAX_CTX:(sq + 1) * MAX_CTX].copy()
            oracle.write_kv_f16(k16[0], ks, 1, s.kv_dim, pos)
            oracle.write_kv_f16(v[0], vs, 1, s.kv_dim, pos)
            attn = oracle.attention(q[0], ks, vs, 1, s.n_head, s.n_kv, s.head_dim, scale, pos).reshape(1, -1)
            h = oracle.add(h, lin(L["wo"], attn))
            hn = oracle.rms_norm(h, L["ffn_norm"], s.eps)
            h = oracle.add(h, lin(L["down"], oracle.gated_act(lin(L["gate"], hn), lin(L["up"], hn))))
        want[sq] = oracle.linear(Q4K, head, oracle.rms_norm(h, out_norm, s.eps), 1, s.hidden, s.vocab)
    for fused, q8 in ((False, False), (True, False), (True, True)):
        step = DecodeStep(backend, s, b, MAX_CTX, dev_layers, on, hd, Q4K, [backend.from_numpy(c) for c in kc], [backend.from_numpy(c) for c in vc])
        step.set_inputs(hidden, positions)
        step.run(int(positions.max()), fused=fused, q8_fused=q8)
        got = backend.download(step.logits, np.float32).reshape(b, s.vocab)
        for sq in range(b):
            assert fx.rel_l2(got[sq], want[sq]) < 1e-3, (fused, q8, sq)
            assert int(np.argmax(got[sq])) == int(np.argmax(want[sq]))
        # the rows written are each sequence's own position
        for li in range(s.n_layer):
            g = backend.download(step.v_cache[li], np.uint16).reshape(vc[li].shape)
            keep = np.ones(g.shape[0], bool)
            keep[[int(positions[0]), MAX_CTX + int(positions[1])]] = False
            np.testing.assert_array_equal(g[keep], vc[li][keep])
            assert (g[~keep] != vc[li][~keep]).any()


def test_paged_caches_give_what_contiguous_caches_give(backend):
    """The same sequences, their cache rows scattered over a pool of 128-row pages through a page table: same logits, same
    tokens, bit for bit, in the fused and the int8-producer form; the new rows land in the right pages."""
    s = LlamaShape(n_layer=2, hidden=512, n_head=4, n_kv=2, head_dim=128, ffn=1024, vocab=400)
    b, ctx = 3, 384  # three pages per sequence
    positions = np.array([300, 129, 5], np.int32)
    layers = []
    for li in range(s.n_layer):
        d = {name: backend.from_numpy(synth.weight(dt, o, i, seed=4000 + 16 * li + t), infr_b200.USAGE_WEIGHTS)
             for t, (name, dt, o, i) in enumerate(s.linears())}
        d["attn_norm"] = backend.from_numpy((1.0 + 0.02 * synth.normal(4100 + li, (s.hidden,))).astype(np.float32))
        d["ffn_norm"] = backend.from_numpy((1.0 + 0.02 * synth.normal(4200 + li, (s.hidden,))).astype(np.float32))
        layers.append(d)
    out_norm = backend.from_numpy((1.0 + 0.02 * synth.normal(4300, (s.hidden,))).astype(np.float32))
    head = backend.from_numpy(synth.weight(Q4K, s.vocab, s.hidden, seed=4301), infr_b200.USAGE_WEIGHTS)
    kc = [synth.normal(80 + li, (b * ctx, s.kv_dim)).astype(np.float16).view(np.uint16) for li in range(s.n_layer)]
    vc = [synth.normal(90 + li, (b * ctx, s.kv_dim)).astype(np.float16).view(np.uint16) for li in range(s.n_layer)]
    hidden = synth.normal(95, (b, s.hidden))
    # page table: sequence sq's page i -> a scrambled page of a pool with spare pages
    n_pages, stride = 13, 4
    perm = np.random.default_rng(7).permutation(n_pages)
    table = np.full((b, stride), -1, np.int32)
    for sq in range(b):
        for i in range(3):
            table[sq, i] = perm[sq * 3 + i]
    table[:, 3] = 10 ** 6  # an entry nobody should need: out of range on purpose

    def pool(c):
        p = np.zeros((n_pages * 128, s.kv_dim), np.uint16)
        for sq in range(b):
            for i in range(3):
                p[table[sq, i] * 128:(table[sq, i] + 1) * 128] = c[sq * ctx + i * 128: sq * ctx + (i + 1) * 128]
        return p
    for fused, q8 in ((True, False), (True, True)):
        ref = DecodeStep(backend, s, b, ctx, layers, out_norm, head, Q4K, [backend.from_numpy(c) for c in kc], [backend.from_numpy(c) for c in vc])
        ref.set_inputs(hidden, positions)
        ref.run(int(positions.max()), fused=fused, q8_fused=q8)
        kp, vp = [backend.from_numpy(pool(c)) for c in kc], [backend.from_numpy(pool(c)) for c in vc]
        pg = DecodeStep(backend, s, b, ctx, layers, out_norm, head, Q4K, kp, vp, pages=(backend.from_numpy(table), stride, n_pages))
        pg.set_inputs(hidden, positions)
        pg.run(int(positions.max()), fused=fused, q8_fused=q8)
        np.testing.assert_array_equal(backend.download(pg.logits, np.uint32), backend.download(ref.logits, np.uint32))
        np.testing.assert_array_equal(backend.download(pg.tok, np.uint32), backend.download(ref.tok, np.uint32))
        for li in range(s.n_layer):
            want = pool(backend.download(ref.v_cache[li], np.uint16).reshape(b * ctx, s.kv_dim))
            np.testing.assert_array_equal(backend.download(vp[li], np.uint16).reshape(n_pages * 128, s.kv_dim), want)
            want_k = pool(backend.download(ref.k_cache[li], np.uint16).reshape(b * ctx, s.kv_dim))
            np.testing.assert_array_equal(backend.download(kp[li], np.uint16).reshape(n_pages * 128, s.kv_dim), want_k)
    with pytest.raises(infr_b200.BackendError):  # a table too narrow for the positions
        backend.attention_paged(ref.q, kp[0], vp[0], backend.from_numpy(table), 2, n_pages, rows=1, pos=300, n_head=s.n_head, n_kv=s.n_kv,
                                head_dim=s.head_dim, scale=1.0, n_seq=b, dst=ref.attn)
