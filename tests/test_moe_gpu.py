"""Op::MoeFfn on the GPU vs the CPU restatement (production int8 path, rows >= 2).

Gates: router logits bit-exact (same FMA order as the reference's `dot`); selected expert ids
identical (near-tie flips would be reported, none are tolerated on these seeds); routing weights
within 1e-6; output within 1e-3 relative L2 of the production CPU path.
"""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from fixtures import Q4K
from infr_b200 import synth

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gemm_backend():
    """Every expert bank on the grouped tensor-memory GEMM, also where the default dispatch (few rows per expert) would
    take the 8-row grouped GEMV."""
    be = infr_b200.CudaBackend(device=0, mmq_kernel=2)
    yield be
    be.close()


_BANKS = {}


def _banks(n_expert, nff, ne, seed):
    key = (n_expert, nff, ne, seed)
    if key not in _BANKS:
        _BANKS[key] = _make_banks(n_expert, nff, ne, seed)
    return _BANKS[key]


def _make_banks(n_expert, nff, ne, seed):
    gate = np.concatenate([synth.weight(Q4K, nff, ne, seed + 3 * e) for e in range(n_expert)])
    up = np.concatenate([synth.weight(Q4K, nff, ne, seed + 3 * e + 1) for e in range(n_expert)])
    down = np.concatenate([synth.weight(Q4K, ne, nff, seed + 3 * e + 2) for e in range(n_expert)])
    return gate, up, down


def _run(backend, x, router, gate, up, down, rows, ne, n_expert, n_used, nff, norm_w=True, scale=1.0, wdt=Q4K, down_dt=None):
    xb = backend.from_numpy(x)
    rb = backend.from_numpy(router)
    gb = backend.from_numpy(gate, infr_b200.USAGE_WEIGHTS)
    ub = backend.from_numpy(up, infr_b200.USAGE_WEIGHTS)
    db = backend.from_numpy(down, infr_b200.USAGE_WEIGHTS)
    dst = backend.alloc(rows * ne * 4)
    ids = backend.alloc(rows * n_used * 4)
    w = backend.alloc(rows * n_used * 4)
    lg = backend.alloc(rows * n_expert * 4)
    backend.moe_ffn(xb, xb, rb, gb, ub, db, dst, rows=rows, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=nff,
                    scale=scale, norm_w=norm_w, sel_ids=ids, sel_w=w, logits=lg, wdt=wdt, down_dt=down_dt)
    out = (backend.download(dst, np.float32).reshape(rows, ne), backend.download(ids, np.int32).reshape(rows, n_used),
           backend.download(w, np.float32).reshape(rows, n_used), backend.download(lg, np.float32).reshape(rows, n_expert))
    for b in (xb, rb, gb, ub, db, dst, ids, w, lg):
        b.close()
    return out


@pytest.mark.parametrize("rows,ne,n_expert,n_used,nff,norm_w,scale", [
    (2, 256, 8, 2, 256, True, 1.0),
    (19, 512, 16, 4, 768, True, 1.0),       # 3-block down projection, ragged 8-row items
    (33, 1024, 32, 8, 256, False, 2.5),     # no renormalisation, scale != 1
    (64, 2048, 128, 8, 768, True, 1.0),     # the Qwen3-30B-A3B layer shape with 64 tokens
    (256, 2048, 128, 8, 768, True, 1.0),    # the MoE configuration itself: 256 tokens, 2048 routed pairs
])
@pytest.mark.parametrize("path", ["default", "grouped-gemm"])
def test_moe_ffn_matches_production_cpu(backend, gemm_backend, oracle, rows, ne, n_expert, n_used, nff, norm_w, scale, path):
    backend = backend if path == "default" else gemm_backend
    gate, up, down = _banks(n_expert, nff, ne, seed=100)
    router = synth.normal(7, (n_expert, ne), 1.0 / np.sqrt(ne))
    x = synth.normal(8, (rows, ne))
    got, ids, w, lg = _run(backend, x, router, gate, up, down, rows, ne, n_expert, n_used, nff, norm_w, scale)
    want, o_ids, o_w, o_lg = oracle.moe_ffn(x, router, gate, up, down, rows=rows, ne=ne, n_expert=n_expert, n_used=n_used,
                                            n_ff_exp=nff, norm_w=norm_w, scale=scale)
    np.testing.assert_array_equal(lg.view(np.uint32), o_lg.view(np.uint32))
    np.testing.assert_array_equal(ids, o_ids)
    np.testing.assert_allclose(w, o_w, rtol=2e-6, atol=1e-7)
    rel = fx.rel_l2(got, want)
    assert rel < 1e-3, rel
    assert np.abs(want).max() > 1e-4


@pytest.mark.parametrize("gu_dt,down_dt", [(Q4K, infr_b200.Q6K), (infr_b200.Q6K, infr_b200.Q6K)], ids=["q4k-gate-up-q6k-down", "all-q6k"])
def test_moe_q6k_expert_banks(backend, oracle, gu_dt, down_dt):
    """Expert banks in Q6_K (`expert_acts_kind` Super, crates/infr-cpu/src/moe.rs:42-53): the Q4_K_M mix keeps the down
    experts in Q6_K.  n_ff_exp = 768 makes the down rows 3 blocks = 630 bytes long (not a multiple of 16)."""
    rows, ne, n_expert, n_used, nff = 21, 512, 8, 2, 768
    gate = np.concatenate([synth.weight(gu_dt, nff, ne, 400 + 3 * e) for e in range(n_expert)])
    up = np.concatenate([synth.weight(gu_dt, nff, ne, 401 + 3 * e) for e in range(n_expert)])
    down = np.concatenate([synth.weight(down_dt, ne, nff, 402 + 3 * e) for e in range(n_expert)])
    router = synth.normal(7, (n_expert, ne), 1.0 / np.sqrt(ne))
    x = synth.normal(8, (rows, ne))
    got, ids, w, lg = _run(backend, x, router, gate, up, down, rows, ne, n_expert, n_used, nff, wdt=gu_dt, down_dt=down_dt)
    want, o_ids, o_w, o_lg = oracle.moe_ffn(x, router, gate, up, down, rows=rows, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=nff,
                                            wdt=gu_dt, down_dt=down_dt)
    np.testing.assert_array_equal(lg.view(np.uint32), o_lg.view(np.uint32))
    np.testing.assert_array_equal(ids, o_ids)
    np.testing.assert_allclose(w, o_w, rtol=2e-6, atol=1e-7)
    assert fx.rel_l2(got, want) < 1e-3
    assert np.abs(want).max() > 1e-4


def test_moe_row_with_a_nan_activation_routes_like_the_cpu(backend, oracle):
    """An overflowed activation makes a row's logits NaN: the CPU's stable sort then keeps index order (experts
    0..k-1) and carries NaN weights; the router must answer the same, in range, and the other rows are untouched."""
    rows, ne, n_expert, n_used, nff = 6, 256, 8, 3, 256
    gate, up, down = _banks(n_expert, nff, ne, seed=31)
    router = synth.normal(7, (n_expert, ne), 1.0 / np.sqrt(ne))
    x = synth.normal(8, (rows, ne))
    x[2, 17] = np.nan
    x[4, 3] = np.inf
    got, ids, w, _ = _run(backend, x, router, gate, up, down, rows, ne, n_expert, n_used, nff)
    want, o_ids, o_w, _ = oracle.moe_ffn(x, router, gate, up, down, rows=rows, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=nff)
    np.testing.assert_array_equal(ids, o_ids)
    np.testing.assert_array_equal(ids[2], np.arange(n_used))
    assert np.isnan(w[2]).all() and np.isnan(o_w[2]).all()
    ok = [0, 1, 3, 5]
    np.testing.assert_allclose(w[ok], o_w[ok], rtol=2e-6, atol=1e-7)
    assert fx.rel_l2(got[ok], want[ok]) < 1e-3
    assert np.isnan(got[2]).all() and np.isnan(want[2]).all()


def test_moe_ties_keep_the_lower_expert_id(backend):
    ne, n_expert, n_used, nff, rows = 256, 8, 3, 256, 2
    gate, up, down = _banks(n_expert, nff, ne, seed=5)
    router = np.zeros((n_expert, ne), np.float32)
    x = synth.normal(3, (rows, ne))
    _, ids, w, _ = _run(backend, x, router, gate, up, down, rows, ne, n_expert, n_used, nff)
    np.testing.assert_array_equal(ids, np.array([[0, 1, 2], [0, 1, 2]], np.int32))
    np.testing.assert_allclose(w, 1 / 3, rtol=1e-6)


def test_moe_through_the_graph_seam_and_skewed_routing(backend, oracle):
    # every token routed to the same two experts: one expert gets many 8-row items
    rows, ne, n_expert, n_used, nff = 40, 256, 8, 2, 256
    gate, up, down = _banks(n_expert, nff, ne, seed=9)
    router = np.zeros((n_expert, ne), np.float32)
    router[5] = 0.05
    router[2] = 0.04
    x = np.abs(synth.normal(4, (rows, ne)))
    g = infr_b200.Graph()
    xid = g.input(rows * ne)
    rid = g.weight(n_expert * ne, infr_b200.F32)
    gid = g.weight(n_expert * nff * ne, Q4K)
    uid = g.weight(n_expert * nff * ne, Q4K)
    did = g.weight(n_expert * ne * nff, Q4K)
    oid = g.output(rows * ne)
    g.moe_ffn(xid, xid, rid, gid, uid, did, oid, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=nff)
    plan = backend.compile(g)
    bufs = {xid: backend.from_numpy(x), rid: backend.from_numpy(router), gid: backend.from_numpy(gate),
            uid: backend.from_numpy(up), did: backend.from_numpy(down), oid: backend.alloc(rows * ne * 4)}
    backend.execute(plan, bufs)
    got = backend.download(bufs[oid], np.float32).reshape(rows, ne)
    want, ids, _, _ = oracle.moe_ffn(x, router, gate, up, down, rows=rows, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=nff)
    assert (ids[:, 0] == 5).all() and (ids[:, 1] == 2).all()
    assert fx.rel_l2(got, want) < 1e-3


def test_moe_single_row_takes_the_f32_activation_path(backend, oracle):
    # rows == 1 (decode): int8_ok is false (crates/infr-cpu/src/lib.rs:2359) -> raw f32 activations,
    # dequantised weight rows and `dot`; compared like reference mode, 1e-5 of the output's magnitude
    ne, n_expert, n_used, nff = 512, 16, 4, 768
    gate, up, down = _banks(n_expert, nff, ne, seed=200)
    router = synth.normal(17, (n_expert, ne), 1.0 / np.sqrt(ne))
    for seed in (1, 2):
        x = synth.normal(seed, (1, ne))
        got, ids, w, lg = _run(backend, x, router, gate, up, down, 1, ne, n_expert, n_used, nff)
        want, o_ids, o_w, o_lg = oracle.moe_ffn(x, router, gate, up, down, rows=1, ne=ne, n_expert=n_expert, n_used=n_used,
                                                n_ff_exp=nff)
        np.testing.assert_array_equal(lg.view(np.uint32), o_lg.view(np.uint32))
        np.testing.assert_array_equal(ids, o_ids)
        assert np.abs(got - want).max() / np.abs(want).max() < 1e-5
        # and it is NOT the int8 path: the production batch path on the same row differs by ~1e-3
        x2 = np.concatenate([x, x])
        prod, _, _, _ = oracle.moe_ffn(x2, router, gate, up, down, rows=2, ne=ne, n_expert=n_expert, n_used=n_used, n_ff_exp=nff)
        assert fx.rel_l2(prod[0], want[0]) > 1e-5


def test_moe_reference_mode_backend(oracle):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    be = infr_b200.CudaBackend(device=0, reference=True)
    try:
        rows, ne, n_expert, n_used, nff = 5, 256, 8, 2, 256
        gate, up, down = _banks(n_expert, nff, ne, seed=300)
        router = synth.normal(27, (n_expert, ne), 1.0 / np.sqrt(ne))
        x = synth.normal(28, (rows, ne))
        got, ids, _, _ = _run(be, x, router, gate, up, down, rows, ne, n_expert, n_used, nff)
        want, o_ids, _, _ = oracle.moe_ffn(x, router, gate, up, down, rows=rows, ne=ne, n_expert=n_expert, n_used=n_used,
                                           n_ff_exp=nff, reference=True)
        np.testing.assert_array_equal(ids, o_ids)
        assert np.abs(got - want).max() / np.abs(want).max() < 1e-5
    finally:
        be.close()


def test_expert_parallel_slices_add_up_to_the_whole_layer(backend):
    """Two 'ranks' run one after the other on the same GPU, each with its half of the expert banks; their outputs
    add up to the unsharded layer's (the per-pair values are the same bits, only the order of the final adds
    differs), and a slice whose experts nobody picked contributes exactly zero."""
    rows, ne, nx, nu, nff = 24, 512, 8, 2, 256
    blk = lambda o, i, seed: synth.weight(Q4K, o, i, seed)
    gate = np.concatenate([blk(nff, ne, 50 + e) for e in range(nx)])
    up = np.concatenate([blk(nff, ne, 70 + e) for e in range(nx)])
    down = np.concatenate([blk(ne, nff, 90 + e) for e in range(nx)])
    router = synth.normal(3, (nx, ne), 1.0 / np.sqrt(ne))
    x = synth.normal(4, (rows, ne))
    per_g, per_d = gate.nbytes // nx, down.nbytes // nx
    xb, rb = backend.from_numpy(x), backend.from_numpy(router)
    kw = dict(rows=rows, ne=ne, n_expert=nx, n_used=nu, n_ff_exp=nff)

    def run(lo, n):
        g = backend.from_numpy(gate[lo * per_g:(lo + n) * per_g], infr_b200.USAGE_WEIGHTS)
        u = backend.from_numpy(up[lo * per_g:(lo + n) * per_g], infr_b200.USAGE_WEIGHTS)
        d = backend.from_numpy(down[lo * per_d:(lo + n) * per_d], infr_b200.USAGE_WEIGHTS)
        dst = backend.alloc(rows * ne * 4)
        backend.moe_ffn(xb, xb, rb, g, u, d, dst, expert_lo=lo, n_local=n, **kw)
        out = backend.download(dst, np.float32).reshape(rows, ne)
        for b in (g, u, d, dst):
            b.close()
        return out

    whole = run(0, nx)
    halves = run(0, nx // 2) + run(nx // 2, nx // 2)
    assert np.abs(whole).max() > 1e-3
    # (a slice with more rows per expert may take the grouped GEMM where the whole layer takes the grouped GEMV: the
    # integer block sums are the same, the f32 sums are rounded in a different order)
    assert fx.rel_l2(halves, whole) < 1e-5
    thirds = run(0, 3) + run(3, 3) + run(6, 2)
    assert fx.rel_l2(thirds, whole) < 1e-5
    with pytest.raises(infr_b200.BackendError):
        run(6, 3)  # leaves [0, n_expert)
