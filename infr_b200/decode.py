"""One decode step of a Llama-family model as the sequence of backend ops the reference emits for it
(crates/infr-llama/src/seam/runner.rs:2641-4493: RmsNorm, Linear q/k/v, Rope, WriteKv, Attention, Linear o, Add,
RmsNorm, Linear gate/up, GatedAct, Linear down, Add, ..., RmsNorm, Linear lm_head, Argmax), issued through the
C ABI.  `fused=True` uses the fused launches (Add+RmsNorm, Rope+Rope+WriteKv+WriteKv) and, for at most 8 rows, the
producers that end in the activation quantiser, so that every Linear is one GEMV launch on int8 codes shared by all
Linears that read the same input; `fused=False` issues the reference's ops one by one.  The batch is `n_seq` independent sequences, one new token each, all at position `pos`,
every sequence with its own f16 KV cache; `set_inputs` also takes one position per sequence (a continuously served batch),
which the rotation, the cache write and the attention then follow per sequence."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

from . import ACT_INT8, Q4K, Q6K, USAGE_ACTIVATIONS, USAGE_WEIGHTS


@dataclass
class LlamaShape:
    n_layer: int = 32
    hidden: int = 4096
    n_head: int = 32
    n_kv: int = 8
    head_dim: int = 128
    ffn: int = 14336
    vocab: int = 128256
    theta: float = 500000.0
    eps: float = 1e-5

    @property
    def q_dim(self) -> int:
        return self.n_head * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.n_kv * self.head_dim

    def linears(self):
        """(name, dtype, out_f, in_f) of one layer in the Q4_K_M mix: attn_v and ffn_down in Q6_K, the rest Q4_K."""
        h, q, kv, ff = self.hidden, self.q_dim, self.kv_dim, self.ffn
        return [("wq", Q4K, q, h), ("wk", Q4K, kv, h), ("wv", Q6K, kv, h), ("wo", Q4K, h, q),
                ("gate", Q4K, ff, h), ("up", Q4K, ff, h), ("down", Q6K, h, ff)]


class DecodeStep:
    """Holds the device buffers of one model replica and issues one decode step.

    `layers` is a list of dicts name -> weight Buffer (the names of LlamaShape.linears plus "attn_norm" and
    "ffn_norm", f32; an optional entry "dtypes": name -> weight format overrides the Q4_K_M mix of LlamaShape.linears
    for that layer, as a model file's per-layer mix does), `head` the lm_head weight (`head_dtype`), `out_norm` the
    output norm.  `k_cache` / `v_cache` are per-layer Buffers holding `n_seq` caches of `max_ctx` rows each."""

    def __init__(self, be, shape: LlamaShape, n_seq: int, max_ctx: int, layers, out_norm, head, head_dtype, k_cache, v_cache,
                 sub=None, reduce=None, argmax: bool = True, pages=None, comm=None):
        """Tensor-parallel use: `shape` holds this rank's share (n_head, n_kv, ffn and vocab divided by the ranks, hidden
        whole), `reduce(buffer, n_floats)` sums the row-parallel Linears' partial results (attention output, FFN down)
        over the ranks in place, `sub` optionally supplies the buffer those results live in (e.g. memory a collective
        library can address), and `argmax=False` leaves the rank's slice of the logits for the caller to gather.
        With `comm` (a connected Comm) a step over at most 8 sequences (32 where the wide GEMV applies) has no exchange kernel at all: the row-parallel
        GEMVs push their partial results to the peers from their epilogues and the norm that follows sums them
        (gemv_q8_push / add_rms_norm_q8_pull); `reduce` stays the fallback for shapes that form does not take."""
        self.be, self.s, self.n_seq, self.max_ctx = be, shape, n_seq, max_ctx
        self.reduce, self.do_argmax, self.comm = reduce, argmax, comm
        # paged caches: pages = (block_table Buffer int32 [n_seq][stride], stride, n_pages); k_cache / v_cache are then
        # per-layer pools of n_pages pages of 128 rows shared by the sequences (fused forms only)
        self.pages = pages
        self.layers, self.out_norm, self.head, self.head_dtype = layers, out_norm, head, head_dtype
        self.k_cache, self.v_cache = k_cache, v_cache
        s, b = shape, n_seq
        f32 = lambda n: be.alloc(b * n * 4, USAGE_ACTIVATIONS)
        self.hidden, self.hn, self.sub = f32(s.hidden), f32(s.hidden), (sub if sub is not None else f32(s.hidden))
        self.q, self.k, self.v, self.k_rot, self.attn = f32(s.q_dim), f32(s.kv_dim), f32(s.kv_dim), f32(s.kv_dim), f32(s.q_dim)
        self.g, self.u, self.act = f32(s.ffn), f32(s.ffn), f32(s.ffn)
        self.logits = f32(s.vocab)
        self.tok = be.alloc(b * 4, USAGE_ACTIVATIONS)
        self.positions = be.alloc(b * 4, USAGE_ACTIVATIONS)
        self.seq_stride = max_ctx * s.kv_dim
        # int8 activations shared by the Linears that read the same input (q/k/v; gate/up): codes, per-256 scales,
        # per-32 and per-16 code sums, sized for the widest input
        kmax = max(s.hidden, s.ffn, s.q_dim)
        self.a_qs = be.alloc(b * kmax, USAGE_ACTIVATIONS)
        self.a_d = be.alloc(b * (kmax // 256) * 4, USAGE_ACTIVATIONS)
        self.a_sums = be.alloc(b * (kmax // 32) * 4, USAGE_ACTIVATIONS)
        self.a_sums16 = be.alloc(b * (kmax // 16) * 4, USAGE_ACTIVATIONS)

    _MIX = {"wq": Q4K, "wk": Q4K, "wv": Q6K, "wo": Q4K, "gate": Q4K, "up": Q4K, "down": Q6K}

    def _dt(self, layer: dict, name: str) -> int:
        return layer.get("dtypes", self._MIX).get(name, self._MIX[name])

    def _q8_formats(self) -> bool:
        """Every Linear takes activations quantised per 256 elements (Q4_K, Q6_K); Q2_0 wants them per 32."""
        names = ("wq", "wk", "wv", "wo", "gate", "up", "down")
        return all(self._dt(L, n) in (Q4K, Q6K) for L in self.layers for n in names) and self.head_dtype in (Q4K, Q6K)

    def _wide_ok(self) -> bool:
        """9..32 sequences: every Linear can take pre-quantised rows (the wide GEMV: Q4_K, or Q6_K rows of whole
        2048-element chunks), so the step keeps its activations in int8 between ops as a step over one sequence does."""
        s = self.s
        if self.n_seq > 32:
            return False
        ins = {"wq": s.hidden, "wk": s.hidden, "wv": s.hidden, "wo": s.q_dim, "gate": s.hidden, "up": s.hidden, "down": s.ffn}
        ok = lambda dt, k: dt == Q4K or (dt == Q6K and k % 2048 == 0)
        return all(ok(self._dt(L, n), k) for L in self.layers for n, k in ins.items()) and ok(self.head_dtype, s.hidden)

    def _push_ok(self, dt: int = None, k: int = None) -> bool:
        """The row-parallel Linear of format `dt` over `k` input columns can push its result from its GEMV's epilogue
        (no arguments: every o and down of the model can)."""
        s = self.s
        if self.comm is None or self.n_seq > 32 or (self.n_seq > 8 and not self._wide_ok()):
            return False
        ok = lambda d_, k_: (d_ == Q4K and k_ % 256 == 0) or (d_ == Q6K and k_ % 2048 == 0)
        if dt is not None:
            return ok(dt, k)
        return all(ok(self._dt(L, "wo"), s.q_dim) and ok(self._dt(L, "down"), s.ffn) for L in self.layers)

    def set_inputs(self, hidden: np.ndarray, pos):
        """pos: one position for every sequence, or one per sequence (sequences that joined the batch at different
        times: `run` then takes the largest)."""
        self.be.upload(self.hidden, np.ascontiguousarray(hidden, np.float32))
        p = np.full(self.n_seq, pos, np.int32) if np.isscalar(pos) else np.ascontiguousarray(pos, np.int32)
        assert p.shape == (self.n_seq,)
        self.uniform_pos = bool((p == p[0]).all())
        self.host_pos = p
        self.be.upload(self.positions, p)

    def run(self, pos: int, fused: bool = True, q8_fused=None) -> int:
        """Enqueues one step (reads self.hidden / self.positions, leaves logits and token ids on the device).
        Returns the number of ops issued."""
        s, b = self.s, self.n_seq
        # sequences at positions of their own: attention reads them from the device, `pos` bounds them
        self._seq_pos = None if getattr(self, "uniform_pos", True) else self.positions
        if q8_fused is None:
            q8_fused = (fused and (b <= 8 or self._wide_ok()) and self._q8_formats() and s.hidden % 256 == 0 and s.ffn % 256 == 0 and
                        s.q_dim % 256 == 0)
        return self._run_q8(pos) if q8_fused else self._run_f32(pos, fused)

    def _run_q8(self, pos: int) -> int:
        """Activations travel between ops as int8 codes wherever the consumer is a Linear (at most 8 rows, or up to 32
        where every Linear can run on the wide GEMV)."""
        be, s, b = self.be, self.s, self.n_seq
        h, ff = s.hidden, s.ffn
        scale = 1.0 / float(np.sqrt(s.head_dim))
        a8 = (self.a_qs, self.a_d, self.a_sums, self.a_sums16)
        gemv = lambda dt, w, y, k, o: be.gemv_q8(dt, w, self.a_qs, self.a_d, self.a_sums, self.a_sums16, y, b, k, o)

        def pair(d1, w1, y1, o1, d2, w2, y2, o2, k):  # two Linears on the same codes: one launch where the formats agree
            if d1 == d2:
                be.gemv_q8_pair(d1, w1, y1, o1, w2, y2, o2, *a8, b, k)
            else:
                gemv(d1, w1, y1, k, o1)
                gemv(d2, w2, y2, k, o2)
        dt = self._dt
        def row_parallel(d_, w, k, norm_w):  # o / down, the sum over the ranks, the residual add, the next norm
            if self._push_ok(d_, k):
                be.gemv_q8_push(self.comm, d_, w, *a8, b, k, h)
                be.add_rms_norm_q8_pull(self.comm, self.hidden, self.hidden, norm_w, b, h, s.eps, *a8)
                return
            gemv(d_, w, self.sub, k, h)
            if self.reduce:
                self.reduce(self.sub, b * h)
            be.add_rms_norm_q8(self.hidden, self.sub, self.hidden, norm_w, b, h, s.eps, *a8)
        be.add_rms_norm_q8(self.hidden, None, None, self.layers[0]["attn_norm"], b, h, s.eps, *a8)
        n = 1
        for li, L in enumerate(self.layers):
            pair(dt(L, "wq"), L["wq"], self.q, s.q_dim, dt(L, "wk"), L["wk"], self.k, s.kv_dim, h)  # q and k: one launch
            gemv(dt(L, "wv"), L["wv"], self.v, h, s.kv_dim)
            if self.pages:
                tbl, stride, n_pages = self.pages
                be.rope_write_kv_paged(self.q, self.k, self.v, self.positions, self.k_cache[li], self.v_cache[li], tbl, stride, n_pages, rows=1,
                                       pos=pos, n_head=s.n_head, n_kv=s.n_kv, head_dim=s.head_dim, theta=s.theta, n_seq=b)
                be.attention_paged(self.q, self.k_cache[li], self.v_cache[li], tbl, stride, n_pages, rows=1, pos=pos, n_head=s.n_head, n_kv=s.n_kv,
                                   head_dim=s.head_dim, scale=scale, n_seq=b, seq_pos=self._seq_pos, q8=a8)
            else:
                be.rope_write_kv(self.q, self.k, self.v, self.positions, self.k_cache[li], self.v_cache[li], rows=1, pos=pos,
                                 n_head=s.n_head, n_kv=s.n_kv, head_dim=s.head_dim, theta=s.theta, n_seq=b, seq_stride=self.seq_stride)
                be.attention_q8(self.q, self.k_cache[li], self.v_cache[li], *a8, rows=1, pos=pos, n_head=s.n_head, n_kv=s.n_kv,
                                head_dim=s.head_dim, scale=scale, n_seq=b, seq_stride=self.seq_stride, seq_pos=self._seq_pos)
            row_parallel(dt(L, "wo"), L["wo"], s.q_dim, L["ffn_norm"])
            pair(dt(L, "gate"), L["gate"], self.g, ff, dt(L, "up"), L["up"], self.u, ff, h)  # gate and up: one launch
            be.gated_act_q8(self.g, self.u, b, ff, *a8)
            nxt = self.layers[li + 1]["attn_norm"] if li + 1 < len(self.layers) else self.out_norm
            row_parallel(dt(L, "down"), L["down"], ff, nxt)
            n += 13  # ops (q/k and gate/up share a launch: 11 launches per layer)
        gemv(self.head_dtype, self.head, self.logits, h, s.vocab)
        if self.do_argmax:
            be.argmax(self.logits, self.tok, s.vocab, b)
        return n + 2

    def _run_f32(self, pos: int, fused: bool) -> int:
        be, s, b = self.be, self.s, self.n_seq
        h, ff = s.hidden, s.ffn
        scale = 1.0 / float(np.sqrt(s.head_dim))
        n = 0
        lin = lambda dt, w, x, y, i, o: be.linear(dt, w, x, y, b, i, o, ACT_INT8)
        # fused and at most 8 rows: quantise an input once and run every Linear that reads it on the shared codes
        # (the same quantiser and GEMV kernels that Linear uses: bit-identical results)
        share = fused and b <= 8 and h % 256 == 0 and ff % 256 == 0

        def lin_many(x, k, outs):
            nonlocal n
            if fused and not share:
                # wider batches: neighbours of one weight format share the quantised (and re-laid) rows
                i = 0
                while i < len(outs):
                    if i + 1 < len(outs) and outs[i][0] == outs[i + 1][0]:
                        (dt, w1, y1, o1), (_, w2, y2, o2) = outs[i], outs[i + 1]
                        be.linear_pair(dt, w1, y1, o1, w2, y2, o2, x, b, k, ACT_INT8)
                        i += 2
                    else:
                        dt, w, y, o = outs[i]
                        lin(dt, w, x, y, k, o)
                        i += 1
                n += len(outs)
                return
            if share:
                be.quantize_q8(256, x, b, k, self.a_qs, self.a_d, self.a_sums, self.a_sums16)
                for dt, w, y, o in outs:
                    be.gemv_q8(dt, w, self.a_qs, self.a_d, self.a_sums, self.a_sums16, y, b, k, o)
            else:
                for dt, w, y, o in outs:
                    lin(dt, w, x, y, k, o)
            n += len(outs)
        be.rms_norm(self.hidden, self.layers[0]["attn_norm"], self.hn, b, h, s.eps)
        n += 1
        for li, L in enumerate(self.layers):
            dt = self._dt
            lin_many(self.hn, h, [(dt(L, "wq"), L["wq"], self.q, s.q_dim), (dt(L, "wk"), L["wk"], self.k, s.kv_dim),
                                  (dt(L, "wv"), L["wv"], self.v, s.kv_dim)])
            if fused and self.pages:
                tbl, stride, n_pages = self.pages
                be.rope_write_kv_paged(self.q, self.k, self.v, self.positions, self.k_cache[li], self.v_cache[li], tbl, stride, n_pages, rows=1,
                                       pos=pos, n_head=s.n_head, n_kv=s.n_kv, head_dim=s.head_dim, theta=s.theta, n_seq=b)
                n += 1
            elif fused:
                be.rope_write_kv(self.q, self.k, self.v, self.positions, self.k_cache[li], self.v_cache[li], rows=1, pos=pos,
                                 n_head=s.n_head, n_kv=s.n_kv, head_dim=s.head_dim, theta=s.theta, n_seq=b, seq_stride=self.seq_stride)
                n += 1
            else:
                if self.pages:
                    raise ValueError("paged caches run in the fused forms (Op::WriteKv addresses one contiguous cache)")
                be.rope(self.k, self.positions, self.k_rot, b, s.n_kv, s.head_dim, s.head_dim, s.theta)
                be.rope(self.q, self.positions, self.q, b, s.n_head, s.head_dim, s.head_dim, s.theta)
                n += 2
                for sq in range(b):  # Op::WriteKv addresses one cache: one call per sequence
                    for src, cache in ((self.k_rot, self.k_cache[li]), (self.v, self.v_cache[li])):
                        row = be.wrap(src.device_ptr() + sq * s.kv_dim * 4, s.kv_dim * 4, USAGE_ACTIVATIONS)
                        one = be.wrap(cache.device_ptr() + sq * self.seq_stride * 2, self.seq_stride * 2, USAGE_ACTIVATIONS)
                        be.write_kv(row, one, 1, s.kv_dim, int(self.host_pos[sq]) if self._seq_pos is not None else pos)
                        row.close()
                        one.close()
                        n += 1
            if self.pages:
                tbl, stride, n_pages = self.pages
                be.attention_paged(self.q, self.k_cache[li], self.v_cache[li], tbl, stride, n_pages, rows=1, pos=pos, n_head=s.n_head, n_kv=s.n_kv,
                                   head_dim=s.head_dim, scale=scale, n_seq=b, seq_pos=self._seq_pos, dst=self.attn)
            else:
                be.attention(self.q, self.k_cache[li], self.v_cache[li], self.attn, rows=1, pos=pos, n_head=s.n_head, n_kv=s.n_kv,
                             head_dim=s.head_dim, scale=scale, n_seq=b, seq_stride=self.seq_stride, seq_pos=self._seq_pos)
            lin(dt(L, "wo"), L["wo"], self.attn, self.sub, s.q_dim, h)
            n += 2
            if self.reduce:
                self.reduce(self.sub, b * h)
            if fused:
                be.add_rms_norm(self.hidden, self.sub, self.hidden, L["ffn_norm"], self.hn, b, h, s.eps)
                n += 1
            else:
                be.add(self.hidden, self.sub, self.hidden, b * h)
                be.rms_norm(self.hidden, L["ffn_norm"], self.hn, b, h, s.eps)
                n += 2
            lin_many(self.hn, h, [(dt(L, "gate"), L["gate"], self.g, ff), (dt(L, "up"), L["up"], self.u, ff)])
            be.gated_act(self.g, self.u, self.act, b, ff)
            lin(dt(L, "down"), L["down"], self.act, self.sub, ff, h)
            n += 2
            if self.reduce:
                self.reduce(self.sub, b * h)
            nxt = self.layers[li + 1]["attn_norm"] if li + 1 < len(self.layers) else self.out_norm
            if fused:
                be.add_rms_norm(self.hidden, self.sub, self.hidden, nxt, self.hn, b, h, s.eps)
                n += 1
            else:
                be.add(self.hidden, self.sub, self.hidden, b * h)
                be.rms_norm(self.hidden, nxt, self.hn, b, h, s.eps)
                n += 2
        lin(self.head_dtype, self.head, self.hn, self.logits, h, s.vocab)
        if self.do_argmax:
            be.argmax(self.logits, self.tok, s.vocab, b)
        return n + 2
