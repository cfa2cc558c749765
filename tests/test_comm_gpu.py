"""infr_cuda_comm_*: the peer-memory all-reduce.  One GPU is all the test run has, and kernels that wait on one
another must not share a GPU, so the multi-rank exchange itself is checked against NCCL by `bench.py --gpus N`
before it times anything; here: the single-rank path (same kernel, world = 1), epochs, and argument checks."""
import numpy as np
import pytest

import infr_b200

pytestmark = pytest.mark.gpu


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
