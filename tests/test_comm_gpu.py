"""infr_cuda_comm_*: the peer-memory all-reduce.  One GPU is all the test run has, and kernels that wait on one
another must not share a GPU, so the multi-rank exchange itself is checked against NCCL by `bench.py --gpus N`
before it times anything; here: the single-rank path (same kernel, world = 1), epochs, and argument checks."""
import numpy as np
import pytest

import infr_b200
from infr_b200 import synth

pytestmark = pytest.mark.gpu

Q4K, Q6K = infr_b200.Q4K, infr_b200.Q6K


def test_single_rank_all_reduce_is_the_identity_and_repeats(backend):
    comm = backend.comm_create(0, 1, 8192)
    x = (np.arange(8192, dtype=np.float32) - 4000.0) / 7.0
    buf = backend.from_numpy(x)
    for n in (4096, 8192, 4, 4096, 4096):  # both parities, several CTAs, a tiny one
        backend.all_reduce(comm, buf, n)
    backend.sync()  # an expired wait would surface here as E_TIMEOUT
    np.testing.assert_array_equal(backend.download(buf, np.float32), x)
    assert len(comm.export()) == 64
    comm.close()
    buf.close()


def test_single_rank_largest_exchange(backend):
    """1 MB, the most one exchange takes (64 CTAs): a batch-32 step of a 4096-wide model sums 512 KB per layer."""
    n = 262144
    comm = backend.comm_create(0, 1, n)
    x = np.cos(np.arange(n, dtype=np.float32))
    buf = backend.from_numpy(x)
    for k in (n, 131072, n):
        backend.all_reduce(comm, buf, k)
    backend.sync()
    np.testing.assert_array_equal(backend.download(buf, np.float32), x)
    comm.close()
    buf.close()


def test_a_peer_that_never_answers_times_out_and_the_context_survives(backend):
    """The bounded wait of the exchange runs out (the second rank's slot is a private buffer nobody writes and the
    poll limit is short): the kernel returns by itself, sync reports E_TIMEOUT once, and the context goes on working."""
    comm = backend.comm_create(0, 2, 4096)
    comm.connect_silent(spin_limit=2048)
    x = np.linspace(-1.0, 1.0, 4096, dtype=np.float32)
    buf = backend.from_numpy(x)
    backend.all_reduce(comm, buf, 4096)
    with pytest.raises(infr_b200.BackendError) as e:
        backend.sync()
    assert e.value.code == infr_b200.E_TIMEOUT
    backend.sync()  # the status word was consumed: the stream itself is healthy
    np.testing.assert_array_equal(backend.download(buf, np.float32), x)  # left unsummed, not garbage
    # an exchange that has all its ranks still works on the same context
    solo = backend.comm_create(0, 1, 4096)
    backend.all_reduce(solo, buf, 4096)
    backend.sync()
    np.testing.assert_array_equal(backend.download(buf, np.float32), x)
    for c in (comm, solo):
        c.close()
    buf.close()


def test_comm_argument_checks(backend):
    for rank, world, n in ((0, 0, 64), (2, 2, 64), (0, 9, 64), (0, 1, 6), (0, 1, 0), (0, 1, (1 << 18) + 4)):
        with pytest.raises(infr_b200.BackendError) as e:
            backend.comm_create(rank, world, n)
        assert e.value.code == infr_b200.E_INVALID
    comm = backend.comm_create(0, 1, 64)
    buf = backend.alloc(64 * 4)
    for n in (6, 128):  # not a multiple of 4; beyond the comm's capacity
        with pytest.raises(infr_b200.BackendError):
            backend.all_reduce(comm, buf, n)
    # a comm of two ranks cannot be used before its peers are connected
    c2 = backend.comm_create(0, 2, 64)
    with pytest.raises(infr_b200.BackendError):
        backend.all_reduce(c2, buf, 64)
    for c in (comm, c2):
        c.close()
    buf.close()


def _q8_set(backend, rows, k):
    return backend.alloc(rows * k), backend.alloc(rows * (k // 256) * 4), backend.alloc(rows * (k // 32) * 4), backend.alloc(rows * (k // 16) * 4)


@pytest.mark.parametrize("dt,in_f,m", [(Q4K, 2048, 1), (Q4K, 1024, 5), (Q6K, 4096, 1), (Q6K, 2048, 8), (Q4K, 4096, 8),
                                       (Q4K, 2048, 12), (Q4K, 4096, 32), (Q6K, 6144, 20)])  # 9..32 rows: the wide GEMV, one or several K chunks
def test_pushed_gemv_and_pulling_norm_match_gemv_all_reduce_norm(backend, dt, in_f, m):
    """The exchange without a kernel of its own (infr_cuda_gemv_q8_push + infr_cuda_add_rms_norm_q8_pull) on one rank:
    the same bits as gemv_q8 -> all_reduce -> add_rms_norm_q8, several pairs in a row (both parities of the staging),
    alternating with stand-alone all-reduces on the same comm."""
    h = 1024
    w = synth.weight(dt, h, in_f, seed=21)
    x, res = synth.normal(22, (m, in_f)), synth.normal(23, (m, h))
    nw = (1.0 + 0.05 * synth.normal(24, (h,))).astype(np.float32)
    wb, xb, nb = backend.from_numpy(w, infr_b200.USAGE_WEIGHTS), backend.from_numpy(x), backend.from_numpy(nw)
    a8 = _q8_set(backend, m, in_f)
    backend.quantize_q8(256, xb, m, in_f, *a8)
    comm = backend.comm_create(0, 1, m * h)
    # reference: the three separate ops
    y, hid_ref = backend.alloc(m * h * 4), backend.from_numpy(res)
    o_ref = _q8_set(backend, m, h)
    backend.gemv_q8(dt, wb, *a8, y, m, in_f, h)
    backend.all_reduce(comm, y, m * h)
    backend.add_rms_norm_q8(hid_ref, y, hid_ref, nb, m, h, 1e-5, *o_ref)
    ref = [backend.download(b, np.uint8) for b in (hid_ref,) + o_ref]
    for _ in range(3):
        hid = backend.from_numpy(res)
        o = _q8_set(backend, m, h)
        backend.gemv_q8_push(comm, dt, wb, *a8, m, in_f, h)
        backend.add_rms_norm_q8_pull(comm, hid, hid, nb, m, h, 1e-5, *o)
        backend.all_reduce(comm, y, m * h)  # a stand-alone exchange between pairs shares the epochs
        backend.sync()
        for got_b, want in zip((hid,) + o, ref):
            np.testing.assert_array_equal(backend.download(got_b, np.uint8), want)
        for b in (hid,) + o:
            b.close()
    comm.close()
    for b in (wb, xb, nb, y, hid_ref) + a8 + o_ref:
        b.close()


def test_push_without_its_peer_times_out_and_call_order_is_checked(backend):
    """A rank whose peer never pushes: the norm's bounded wait runs out, the row keeps a + nothing, sync reports
    E_TIMEOUT once and the context goes on.  The pair's order is checked on the host."""
    m, in_f, h = 1, 1024, 512
    wb = backend.from_numpy(synth.weight(Q4K, h, in_f, seed=31), infr_b200.USAGE_WEIGHTS)
    xb, nb = backend.from_numpy(synth.normal(32, (m, in_f))), backend.from_numpy(np.ones(h, np.float32))
    res = synth.normal(33, (m, h))
    hid = backend.from_numpy(res)
    a8, o = _q8_set(backend, m, in_f), _q8_set(backend, m, h)
    backend.quantize_q8(256, xb, m, in_f, *a8)
    comm = backend.comm_create(0, 2, m * h)
    comm.connect_silent(spin_limit=2048)
    with pytest.raises(infr_b200.BackendError):  # nothing was pushed
        backend.add_rms_norm_q8_pull(comm, hid, hid, nb, m, h, 1e-5, *o)
    backend.gemv_q8_push(comm, Q4K, wb, *a8, m, in_f, h)
    with pytest.raises(infr_b200.BackendError):  # the first result has not been consumed
        backend.gemv_q8_push(comm, Q4K, wb, *a8, m, in_f, h)
    with pytest.raises(infr_b200.BackendError):  # nor may another exchange come between the two halves
        backend.all_reduce(comm, hid, m * h)
    backend.add_rms_norm_q8_pull(comm, hid, hid, nb, m, h, 1e-5, *o)
    with pytest.raises(infr_b200.BackendError) as e:
        backend.sync()
    assert e.value.code == infr_b200.E_TIMEOUT
    backend.sync()
    np.testing.assert_array_equal(backend.download(hid, np.float32).reshape(m, h), res)  # nothing was added
    with pytest.raises(infr_b200.BackendError):  # shapes the matrix-unit GEMV does not take are refused, not walked
        backend.gemv_q8_push(comm, Q6K, wb, *a8, m, in_f, h)
    comm.close()
    for b in (wb, xb, nb, hid) + a8 + o:
        b.close()
