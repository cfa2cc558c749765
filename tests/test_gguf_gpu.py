"""A model file end to end: a small Llama-shaped GGUF (per-layer format mix as model files have it: attn_v and
ffn_down in Q6_K in one layer, Q4_K in the other) is read by the library's GGUF reader, uploaded straight from the
mapping, and run as a decode step; the logits and the token are those of the same weights handed over directly, and
within the parity bar of the CPU op sequence.  q | k | v placed back to back give the `w_off` slices of a fused-QKV
Linear (crates/infr-llama/src/seam/runner.rs:3445-3461)."""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from infr_b200 import Q4K, Q6K, synth
from infr_b200.decode import DecodeStep, LlamaShape
from infr_b200.gguf_file import GGML_F32, GGML_Q4_K, GGML_Q6_K, load_llama
import gguf_writer as gw

pytestmark = pytest.mark.gpu

S = LlamaShape(n_layer=2, hidden=512, n_head=4, n_kv=2, head_dim=128, ffn=1024, vocab=600, theta=10000.0, eps=1e-6)
N_SEQ, MAX_CTX, POS = 2, 40, 21
GG = {Q4K: GGML_Q4_K, Q6K: GGML_Q6_K}
LONG = {"wq": "attn_q", "wk": "attn_k", "wv": "attn_v", "wo": "attn_output", "gate": "ffn_gate", "up": "ffn_up", "down": "ffn_down"}


def _weights():
    layers = []
    for li in range(S.n_layer):
        mix = {"wq": Q4K, "wk": Q4K, "wv": Q6K if li == 0 else Q4K, "wo": Q4K, "gate": Q4K, "up": Q4K, "down": Q6K if li == 0 else Q4K}
        L = {"dtypes": mix}
        for t, (name, _, o, i) in enumerate(S.linears()):
            L[name] = (mix[name], synth.weight(mix[name], o, i, seed=500 + 16 * li + t), o, i)
        L["attn_norm"] = (1.0 + 0.05 * synth.normal(600 + li, (S.hidden,))).astype(np.float32)
        L["ffn_norm"] = (1.0 + 0.05 * synth.normal(700 + li, (S.hidden,))).astype(np.float32)
        layers.append(L)
    out_norm = (1.0 + 0.05 * synth.normal(800, (S.hidden,))).astype(np.float32)
    head = synth.weight(Q6K, S.vocab, S.hidden, seed=801)
    embd = synth.normal(802, (S.vocab, S.hidden)).astype(np.float32)
    return layers, out_norm, head, embd


def _write(path, layers, out_norm, head, embd):
    meta = [("general.architecture", gw.STR, "llama"), ("llama.block_count", gw.U32, S.n_layer), ("llama.embedding_length", gw.U32, S.hidden),
            ("llama.attention.head_count", gw.U32, S.n_head), ("llama.attention.head_count_kv", gw.U32, S.n_kv),
            ("llama.feed_forward_length", gw.U32, S.ffn), ("llama.rope.freq_base", gw.F32, S.theta),
            ("llama.attention.layer_norm_rms_epsilon", gw.F32, S.eps), ("llama.context_length", gw.U32, 4096)]
    tensors = [("token_embd.weight", (S.hidden, S.vocab), GGML_F32, embd)]
    for li, L in enumerate(layers):
        for name, long in LONG.items():
            dt, w, o, i = L[name]
            tensors.append((f"blk.{li}.{long}.weight", (i, o), GG[dt], w))
        tensors.append((f"blk.{li}.attn_norm.weight", (S.hidden,), GGML_F32, L["attn_norm"]))
        tensors.append((f"blk.{li}.ffn_norm.weight", (S.hidden,), GGML_F32, L["ffn_norm"]))
    tensors += [("output_norm.weight", (S.hidden,), GGML_F32, out_norm), ("output.weight", (S.hidden, S.vocab), GGML_Q6_K, head)]
    gw.write_gguf(path, meta, tensors)


def test_a_model_file_runs_a_decode_step(backend, oracle, tmp_path):
    layers, out_norm, head, embd = _weights()
    p = tmp_path / "tiny-llama.gguf"
    _write(p, layers, out_norm, head, embd)
    m = load_llama(backend, str(p))
    s = m.shape
    assert (s.n_layer, s.hidden, s.n_head, s.n_kv, s.head_dim, s.ffn, s.vocab) == (S.n_layer, S.hidden, S.n_head, S.n_kv, S.head_dim, S.ffn, S.vocab)
    assert abs(s.theta - S.theta) < 1e-3 and abs(s.eps - S.eps) < 1e-12 and m.head_dtype == Q6K
    assert m.layers[0]["dtypes"]["wv"] == Q6K and m.layers[1]["dtypes"]["wv"] == Q4K
    tokens = [17, 403]
    hidden = m.embed(tokens)
    np.testing.assert_array_equal(hidden, embd[tokens])

    kc = [synth.normal(30 + li, (N_SEQ * MAX_CTX, S.kv_dim)).astype(np.float16).view(np.uint16) for li in range(S.n_layer)]
    vc = [synth.normal(40 + li, (N_SEQ * MAX_CTX, S.kv_dim)).astype(np.float16).view(np.uint16) for li in range(S.n_layer)]

    def run(dev_layers, norm_b, head_b, head_dt):
        kcb, vcb = [backend.from_numpy(c) for c in kc], [backend.from_numpy(c) for c in vc]
        step = DecodeStep(backend, s, N_SEQ, MAX_CTX, dev_layers, norm_b, head_b, head_dt, kcb, vcb)
        step.set_inputs(hidden, POS)
        step.run(POS, fused=True)
        return backend.download(step.logits, np.float32).reshape(N_SEQ, s.vocab), backend.download(step.tok, np.uint32)
    got_logits, got_tok = run(m.layers, m.out_norm, m.head, m.head_dtype)

    # the same weights handed over directly
    direct = []
    for L in layers:
        d = {name: backend.from_numpy(L[name][1], infr_b200.USAGE_WEIGHTS) for name in LONG}
        d["attn_norm"], d["ffn_norm"], d["dtypes"] = backend.from_numpy(L["attn_norm"]), backend.from_numpy(L["ffn_norm"]), L["dtypes"]
        direct.append(d)
    want_logits, want_tok = run(direct, backend.from_numpy(out_norm), backend.from_numpy(head, infr_b200.USAGE_WEIGHTS), Q6K)
    np.testing.assert_array_equal(got_logits.view(np.uint32), want_logits.view(np.uint32))
    np.testing.assert_array_equal(got_tok, want_tok)

    # and the CPU op sequence on the same weights
    o, b = oracle, N_SEQ
    pos = np.full(b, POS, np.float32)
    lin = lambda w, x: o.linear(w[0], w[1], x, b, w[3], w[2])
    h = hidden.copy()
    kcs, vcs = [c.copy() for c in kc], [c.copy() for c in vc]
    for li, L in enumerate(layers):
        hn = o.rms_norm(h, L["attn_norm"], S.eps)
        q, k, v = lin(L["wq"], hn), lin(L["wk"], hn), lin(L["wv"], hn)
        k16 = o.rope(k, pos, S.n_kv, S.head_dim, S.head_dim, S.theta)
        q = o.rope(q, pos, S.n_head, S.head_dim, S.head_dim, S.theta)
        attn = np.empty((b, S.q_dim), np.float32)
        for sq in range(b):
            ks, vs = kcs[li][sq * MAX_CTX:(sq + 1) * MAX_CTX], vcs[li][sq * MAX_CTX:(sq + 1) * MAX_CTX]
            o.write_kv_f16(k16[sq], ks, 1, S.kv_dim, POS)
            o.write_kv_f16(v[sq], vs, 1, S.kv_dim, POS)
            attn[sq] = o.attention(q[sq], ks, vs, 1, S.n_head, S.n_kv, S.head_dim, 1.0 / np.sqrt(S.head_dim), POS)
        h = o.add(h, lin(L["wo"], attn))
        hn = o.rms_norm(h, L["ffn_norm"], S.eps)
        h = o.add(h, lin(L["down"], o.gated_act(lin(L["gate"], hn), lin(L["up"], hn))))
    cpu_logits = o.linear(Q6K, head, o.rms_norm(h, out_norm, S.eps), b, S.hidden, S.vocab)
    assert fx.rel_l2(got_logits, cpu_logits) < 1e-3
    np.testing.assert_array_equal(got_tok, o.argmax(cpu_logits, S.vocab))

    # fused QKV: layer 1 has q, k, v in one format, back to back in one buffer; Linear with w_off reads the slices
    assert m.fused_qkv[0] is None and m.fused_qkv[1] is not None
    buf, dt = m.fused_qkv[1]
    x = synth.normal(5, (3, S.hidden))
    xb = backend.from_numpy(x)
    off = 0
    for name, rows in (("wq", S.q_dim), ("wk", S.kv_dim), ("wv", S.kv_dim)):
        yb = backend.alloc(3 * rows * 4)
        backend.linear(dt, buf, xb, yb, 3, S.hidden, rows, w_off=off * S.hidden)
        got = backend.download(yb, np.float32).reshape(3, rows)
        want = o.linear(dt, layers[1][name][1], x, 3, S.hidden, rows)
        assert fx.rel_l2(got, want) < 1e-5
        off += rows
        yb.close()
    m.gguf.close()
