"""infr_cuda_execute keeps a plan's launch sequence as a CUDA graph from its second run on the same buffers.  The replay
must read what the buffers hold NOW, must not outlive the things it was captured with (other buffers, a reallocated
context scratch), and must leave a caller's own capture alone."""
import numpy as np
import pytest

import infr_b200
from infr_b200 import Q4K, Q6K, synth

pytestmark = pytest.mark.gpu


def _plan(be, m, in_f, mid, out_f):
    """x -> Linear (Q4_K) -> Add with a bias row -> Linear (Q6_K): three launches and an Internal handle."""
    g = infr_b200.Graph()
    x, w1, w2, bias, y = g.input(m * in_f), g.weight(mid * in_f, Q4K), g.weight(out_f * mid, Q6K), g.input(m * mid), g.output(m * out_f)
    t, u = g.internal(m * mid), g.internal(m * mid)
    g.linear(x, w1, t, m, in_f, mid)
    g.add(t, bias, u, m * mid)
    g.linear(u, w2, y, m, mid, out_f)
    return be.compile(g), (x, w1, w2, bias, y)


def _direct(be, xb, w1b, w2b, bb, m, in_f, mid, out_f):
    t, u, y = be.alloc(m * mid * 4), be.alloc(m * mid * 4), be.alloc(m * out_f * 4)
    be.linear(Q4K, w1b, xb, t, m, in_f, mid)
    be.add(t, bb, u, m * mid)
    be.linear(Q6K, w2b, u, y, m, mid, out_f)
    out = be.download(y, np.float32)
    for b in (t, u, y):
        b.close()
    return out


def test_replayed_plan_reads_current_data_and_follows_its_bindings(backend):
    be, (m, in_f, mid, out_f) = backend, (3, 1024, 2048, 320)
    plan, (x, w1, w2, bias, y) = _plan(be, m, in_f, mid, out_f)
    w1b = be.from_numpy(synth.weight(Q4K, mid, in_f, seed=1), infr_b200.USAGE_WEIGHTS)
    w2b = be.from_numpy(synth.weight(Q6K, out_f, mid, seed=2), infr_b200.USAGE_WEIGHTS)
    bb = be.from_numpy(synth.normal(3, (m, mid)))
    xb, yb = be.alloc(m * in_f * 4), be.alloc(m * out_f * 4)
    bound = be.bind({x: xb, w1: w1b, w2: w2b, bias: bb, y: yb})
    l0 = be.launch_count()
    per_run = None
    for k in range(5):  # op by op, captured, replayed x3 - each on fresh input
        xs = synth.normal(10 + k, (m, in_f))
        be.upload(xb, xs)
        be.execute(plan, bound)
        got = be.download(yb, np.float32)
        n = be.launch_count() - l0
        want = _direct(be, xb, w1b, w2b, bb, m, in_f, mid, out_f)
        l0 = be.launch_count()
        np.testing.assert_array_equal(got, want)
        per_run = n if per_run is None else per_run
        assert n == per_run  # a replay claims the launches it makes, no more
    # other buffers for the same handles: not the captured graph's
    xb2, yb2 = be.from_numpy(synth.normal(20, (m, in_f))), be.alloc(m * out_f * 4)
    be.execute(plan, {x: xb2, w1: w1b, w2: w2b, bias: bb, y: yb2})
    np.testing.assert_array_equal(be.download(yb2, np.float32), _direct(be, xb2, w1b, w2b, bb, m, in_f, mid, out_f))
    # the context scratch grows (a wide Linear elsewhere): graphs captured before it are dropped, not replayed
    big_w = be.from_numpy(synth.weight(Q4K, 512, 16384, seed=4), infr_b200.USAGE_WEIGHTS)
    big_x, big_y = be.from_numpy(synth.normal(5, (64, 16384))), be.alloc(64 * 512 * 4)
    be.linear(Q4K, big_w, big_x, big_y, 64, 16384, 512)
    for k in range(3):
        be.upload(xb, synth.normal(30 + k, (m, in_f)))
        be.execute(plan, bound)
        np.testing.assert_array_equal(be.download(yb, np.float32), _direct(be, xb, w1b, w2b, bb, m, in_f, mid, out_f))
    # inside the caller's own capture the ops are issued directly, and the captured graph is the caller's
    be.upload(xb, synth.normal(40, (m, in_f)))
    want = _direct(be, xb, w1b, w2b, bb, m, in_f, mid, out_f)
    be.capture_begin()
    be.execute(plan, bound)
    graph = be.capture_end()
    graph.launch()
    np.testing.assert_array_equal(be.download(yb, np.float32), want)
    graph.close()
    plan.close()
    for b in (w1b, w2b, bb, xb, yb, xb2, yb2, big_w, big_x, big_y):
        b.close()
