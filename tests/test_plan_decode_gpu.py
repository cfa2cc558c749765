"""A decode step as the reference emits it — the ordered op list of crates/infr-llama/src/seam/runner.rs:2641-4493 for a
Llama-family model: RmsNorm, Linear q/k/v, Rope(k), Rope(q), WriteKv(k), WriteKv(v), Attention, Linear o, Add, RmsNorm,
Linear gate/up, GatedAct, Linear down, Add, ..., RmsNorm, Linear lm_head, Argmax — through infr_cuda_compile /
infr_cuda_execute, against (a) the same step issued call by call through the direct entry points (same bits: the plan
only groups launches) and (b) the CPU restatement of the op sequence (same argmax, 1e-3 relative L2)."""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from infr_b200 import Q4K, synth
from infr_b200.decode import DecodeStep, LlamaShape

pytestmark = pytest.mark.gpu

SHAPE = LlamaShape(n_layer=2, hidden=512, n_head=4, n_kv=2, head_dim=128, ffn=1024, vocab=1000)
MAX_CTX, POS = 48, 37


def _model(seed0=2000):
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
    kc = [synth.normal(9 + 2 * li, (MAX_CTX, s.kv_dim)).astype(np.float16).view(np.uint16) for li in range(s.n_layer)]
    vc = [synth.normal(10 + 2 * li, (MAX_CTX, s.kv_dim)).astype(np.float16).view(np.uint16) for li in range(s.n_layer)]
    return layers, out_norm, head, kc, vc


def build_graph(s: LlamaShape, rows: int, pos: int, max_ctx: int, layer_dtypes):
    """The reference's emission order (generate_dense_backend with the conservative capability set).  Returns the
    graph and the handle ids by role."""
    g = infr_b200.Graph()
    ids = {"hidden": g.input(rows * s.hidden), "positions": g.input(rows, infr_b200.I32), "layers": []}
    h, qd, kvd, ff = s.hidden, s.q_dim, s.kv_dim, s.ffn
    hn, q, k, v, k16 = (g.internal(rows * n) for n in (h, qd, kvd, kvd, kvd))
    attn, sub, gb, ub, act = (g.internal(rows * n) for n in (qd, h, ff, ff, ff))
    scale = 1.0 / float(np.sqrt(s.head_dim))
    for li in range(s.n_layer):
        L = {"attn_norm": g.weight(h, infr_b200.F32), "ffn_norm": g.weight(h, infr_b200.F32)}
        for name, dt, o, i in layer_dtypes:
            L[name] = g.weight(o * i, dt)
        L["k_cache"] = g.input(max_ctx * kvd, infr_b200.F16)
        L["v_cache"] = g.input(max_ctx * kvd, infr_b200.F16)
        ids["layers"].append(L)
        dts = {name: dt for name, dt, _, _ in layer_dtypes}
        g.rms_norm(ids["hidden"], L["attn_norm"], hn, rows, h, s.eps)
        g.linear(hn, L["wq"], q, rows, h, qd)
        g.linear(hn, L["wk"], k, rows, h, kvd)
        g.linear(hn, L["wv"], v, rows, h, kvd)
        g.rope(k, ids["positions"], k16, rows, s.n_kv, s.head_dim, s.head_dim, s.theta)
        g.rope(q, ids["positions"], q, rows, s.n_head, s.head_dim, s.head_dim, s.theta)
        g.write_kv(k16, L["k_cache"], rows, kvd, pos)
        g.write_kv(v, L["v_cache"], rows, kvd, pos)
        g.attention(q, L["k_cache"], L["v_cache"], attn, rows, pos + rows, s.n_head, s.n_kv, s.head_dim, scale, pos)
        g.linear(attn, L["wo"], sub, rows, qd, h)
        g.add(ids["hidden"], sub, ids["hidden"], rows * h)
        g.rms_norm(ids["hidden"], L["ffn_norm"], hn, rows, h, s.eps)
        g.linear(hn, L["gate"], gb, rows, h, ff)
        g.linear(hn, L["up"], ub, rows, h, ff)
        g.gated_act(gb, ub, act, rows, ff)
        g.linear(act, L["down"], sub, rows, ff, h)
        g.add(ids["hidden"], sub, ids["hidden"], rows * h)
        assert dts  # (dtypes travel in the weight declarations)
    ids["out_norm"] = g.weight(h, infr_b200.F32)
    ids["head"] = g.weight(s.vocab * h, Q4K)
    g.rms_norm(ids["hidden"], ids["out_norm"], hn, rows, h, s.eps)
    lm_in = hn
    if rows > 1:  # logits of the last row only (runner.rs:4436-4450)
        lm_in = g.internal(h)
        g.copy(hn, (rows - 1) * h, lm_in, 0, h)
    ids["logits"] = g.output(s.vocab)
    ids["tok"] = g.output(1, infr_b200.I32)
    g.linear(lm_in, ids["head"], ids["logits"], 1, h, s.vocab)
    g.argmax(ids["logits"], ids["tok"], s.vocab, 1)
    return g, ids


def _upload(backend, layers, out_norm, head, kc, vc):
    s = SHAPE
    dev = []
    for L in layers:
        d = {name: backend.from_numpy(L[name][1], infr_b200.USAGE_WEIGHTS) for name, *_ in s.linears()}
        d["attn_norm"], d["ffn_norm"] = backend.from_numpy(L["attn_norm"]), backend.from_numpy(L["ffn_norm"])
        dev.append(d)
    return (dev, backend.from_numpy(out_norm), backend.from_numpy(head, infr_b200.USAGE_WEIGHTS), [backend.from_numpy(c) for c in kc],
            [backend.from_numpy(c) for c in vc])


def _bind(ids, dev_layers, out_norm_b, head_b, kcb, vcb, hidden_b, pos_b, logits_b, tok_b):
    bind = {ids["hidden"]: hidden_b, ids["positions"]: pos_b, ids["out_norm"]: out_norm_b, ids["head"]: head_b, ids["logits"]: logits_b,
            ids["tok"]: tok_b}
    for li, L in enumerate(ids["layers"]):
        for name in ("attn_norm", "ffn_norm", "wq", "wk", "wv", "wo", "gate", "up", "down"):
            bind[L[name]] = dev_layers[li][name]
        bind[L["k_cache"]], bind[L["v_cache"]] = kcb[li], vcb[li]
    return bind


def test_decode_graph_through_compile_execute_equals_direct_calls_and_cpu(backend, oracle):
    s = SHAPE
    layers, out_norm, head, kc, vc = _model()
    hidden = synth.normal(78, (1, s.hidden))
    # (a) call by call through the direct entry points, fused launches
    dev_layers, onb, hb, kcb, vcb = _upload(backend, layers, out_norm, head, kc, vc)
    step = DecodeStep(backend, s, 1, MAX_CTX, dev_layers, onb, hb, Q4K, kcb, vcb)
    step.set_inputs(hidden, POS)
    step.run(POS, fused=True)
    want_logits = backend.download(step.logits, np.float32)
    want_tok = backend.download(step.tok, np.uint32)
    want_k = [backend.download(c, np.uint16) for c in kcb]
    want_v = [backend.download(c, np.uint16) for c in vcb]
    # (b) the op list through the graph seam, on fresh copies of the caches
    g, ids = build_graph(s, 1, POS, MAX_CTX, s.linears())
    plan = backend.compile(g)
    kcb2, vcb2 = [backend.from_numpy(c) for c in kc], [backend.from_numpy(c) for c in vc]
    hidden_b = backend.from_numpy(hidden)
    pos_b = backend.from_numpy(np.full(1, POS, np.int32))
    logits_b, tok_b = backend.alloc(s.vocab * 4), backend.alloc(4)
    l0 = backend.launch_count()
    backend.execute(plan, _bind(ids, dev_layers, onb, hb, kcb2, vcb2, hidden_b, pos_b, logits_b, tok_b))
    launches = backend.launch_count() - l0
    got_logits = backend.download(logits_b, np.float32)
    got_tok = backend.download(tok_b, np.uint32)
    np.testing.assert_array_equal(got_logits.view(np.uint32), want_logits.view(np.uint32))
    np.testing.assert_array_equal(got_tok, want_tok)
    for li in range(s.n_layer):
        np.testing.assert_array_equal(backend.download(kcb2[li], np.uint16), want_k[li])
        np.testing.assert_array_equal(backend.download(vcb2[li], np.uint16), want_v[li])
    # the plan groups launches: fewer kernels than the 17 ops per layer it was given
    assert launches <= 15 * s.n_layer + 4, launches
    # the mutated f32 Input is visible in its bound buffer (graph_input_inplace): hidden now holds the residual stream
    assert not np.array_equal(backend.download(hidden_b, np.float32), hidden.ravel())

    # (c) against the CPU restatement of the same op sequence
    o = oracle
    hid = hidden.copy()
    pos = np.full(1, POS, np.float32)
    scale = 1.0 / np.sqrt(s.head_dim)
    okc, ovc = [c.copy() for c in kc], [c.copy() for c in vc]
    lin = lambda w, x: o.linear(w[0], w[1], x, 1, w[3], w[2])
    for li, L in enumerate(layers):
        hn = o.rms_norm(hid, L["attn_norm"], s.eps)
        q, k, v = lin(L["wq"], hn), lin(L["wk"], hn), lin(L["wv"], hn)
        k16 = o.rope(k, pos, s.n_kv, s.head_dim, s.head_dim, s.theta)
        q = o.rope(q, pos, s.n_head, s.head_dim, s.head_dim, s.theta)
        o.write_kv_f16(k16[0], okc[li], 1, s.kv_dim, POS)
        o.write_kv_f16(v[0], ovc[li], 1, s.kv_dim, POS)
        attn = o.attention(q[0], okc[li], ovc[li], 1, s.n_head, s.n_kv, s.head_dim, scale, POS).reshape(1, -1)
        hid = o.add(hid, lin(L["wo"], attn))
        hn = o.rms_norm(hid, L["ffn_norm"], s.eps)
        act = o.gated_act(lin(L["gate"], hn), lin(L["up"], hn))
        hid = o.add(hid, lin(L["down"], act))
    hn = o.rms_norm(hid, out_norm, s.eps)
    cpu_logits = o.linear(Q4K, head, hn, 1, s.hidden, s.vocab)
    assert fx.rel_l2(got_logits, cpu_logits.ravel()) < 1e-3
    assert int(got_tok[0]) == int(o.argmax(cpu_logits, s.vocab)[0])
    plan.close()


def test_prefill_rows_of_one_sequence_through_the_graph(backend):
    """rows = 3 consecutive positions of one sequence (the reference's batch semantics): the plan's grouped launches
    against the same ops issued one by one through the direct entry points."""
    s, rows = SHAPE, 3
    layers, out_norm, head, kc, vc = _model(seed0=2100)
    hidden = synth.normal(79, (rows, s.hidden))
    dev_layers, onb, hb, kcb, vcb = _upload(backend, layers, out_norm, head, kc, vc)
    g, ids = build_graph(s, rows, POS, MAX_CTX, s.linears())
    plan = backend.compile(g)
    hidden_b = backend.from_numpy(hidden)
    pos_b = backend.from_numpy(np.arange(POS, POS + rows, dtype=np.int32))
    logits_b, tok_b = backend.alloc(s.vocab * 4), backend.alloc(4)
    backend.execute(plan, _bind(ids, dev_layers, onb, hb, kcb, vcb, hidden_b, pos_b, logits_b, tok_b))
    got = backend.download(logits_b, np.float32)
    got_k = [backend.download(c, np.uint16) for c in kcb]

    # one by one
    be = backend
    kcb2, vcb2 = [be.from_numpy(c) for c in kc], [be.from_numpy(c) for c in vc]
    f32 = lambda n: be.alloc(rows * n * 4)
    h, qd, kvd, ff = s.hidden, s.q_dim, s.kv_dim, s.ffn
    hid, hn, q, k, v, k16, attn, sub, gb, ub, act = (f32(n) for n in (h, h, qd, kvd, kvd, kvd, qd, h, ff, ff, ff))
    be.upload(hid, hidden)
    scale = 1.0 / float(np.sqrt(s.head_dim))
    for li, L in enumerate(dev_layers):
        dts = {name: dt for name, dt, _, _ in s.linears()}
        be.rms_norm(hid, L["attn_norm"], hn, rows, h, s.eps)
        be.linear_pair(dts["wq"], L["wq"], q, qd, L["wk"], k, kvd, hn, rows, h)  # the plan pairs q / k and gate / up too
        be.linear(dts["wv"], L["wv"], hn, v, rows, h, kvd)
        be.rope(k, pos_b, k16, rows, s.n_kv, s.head_dim, s.head_dim, s.theta)
        be.rope(q, pos_b, q, rows, s.n_head, s.head_dim, s.head_dim, s.theta)
        be.write_kv(k16, kcb2[li], rows, kvd, POS)
        be.write_kv(v, vcb2[li], rows, kvd, POS)
        be.attention(q, kcb2[li], vcb2[li], attn, rows=rows, pos=POS, n_head=s.n_head, n_kv=s.n_kv, head_dim=s.head_dim, scale=scale)
        be.linear(dts["wo"], L["wo"], attn, sub, rows, qd, h)
        be.add(hid, sub, hid, rows * h)
        be.rms_norm(hid, L["ffn_norm"], hn, rows, h, s.eps)
        be.linear_pair(dts["gate"], L["gate"], gb, ff, L["up"], ub, ff, hn, rows, h)
        be.gated_act(gb, ub, act, rows, ff)
        be.linear(dts["down"], L["down"], act, sub, rows, ff, h)
        be.add(hid, sub, hid, rows * h)
    be.rms_norm(hid, onb, hn, rows, h, s.eps)
    last = be.wrap(hn.device_ptr() + (rows - 1) * h * 4, h * 4, infr_b200.USAGE_ACTIVATIONS)
    want_b = be.alloc(s.vocab * 4)
    be.linear(Q4K, hb, last, want_b, 1, h, s.vocab)
    want = be.download(want_b, np.float32)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    for li in range(s.n_layer):
        np.testing.assert_array_equal(got_k[li], be.download(kcb2[li], np.uint16))
    plan.close()


def test_compile_rejects_what_this_backend_does_not_run(backend):
    g = infr_b200.Graph()
    x, p, d = g.input(256), g.input(1, infr_b200.I32), g.internal(256)
    g.rope(x, p, d, 1, 2, 128, 128, 10000.0, backward=True)
    with pytest.raises(infr_b200.BackendError) as e:
        backend.compile(g)
    assert e.value.code == infr_b200.E_UNSUPPORTED and "backward" in str(e.value)
    g = infr_b200.Graph()
    a, b, c = g.input(1024), g.input(1024), g.internal(1024)
    g.gated_act(a, b, c, 1, 1024, act=1)  # GELU
    with pytest.raises(infr_b200.BackendError) as e:
        backend.compile(g)
    assert e.value.code == infr_b200.E_UNSUPPORTED
    g = infr_b200.Graph()
    g._op(99, (0, 0, 0))
    with pytest.raises(infr_b200.BackendError) as e:
        backend.compile(g)
    assert e.value.code == infr_b200.E_UNSUPPORTED


def test_internal_handles_read_as_zero_until_written(backend):
    """exec.rs:53-92: Internal scratch is zeroed before the walk.  Add reads an Internal nobody wrote: it must see zeros
    even though the pool hands out a block an earlier plan has dirtied."""
    n = 4096
    for _ in range(2):
        g = infr_b200.Graph()
        a, z, out, junk = g.input(n), g.internal(n), g.output(n), g.internal(n)
        g.add(a, z, out, n)      # z is read before anything writes it
        g.add(a, a, junk, n)     # dirties a pool block for the next round
        plan = backend.compile(g)
        av = synth.normal(5, (n,))
        ab, ob = backend.from_numpy(av), backend.alloc(n * 4)
        backend.execute(plan, {a: ab, out: ob})
        np.testing.assert_array_equal(backend.download(ob, np.float32), av)
        plan.close()
