"""infr_cuda_wrap / infr_cuda_stream: ops on device memory the caller owns, on a stream the caller can share."""
import numpy as np
import pytest

import fixtures as fx
import infr_b200
from fixtures import Q4K
from infr_b200 import synth

pytestmark = pytest.mark.gpu


def test_linear_on_wrapped_memory_matches_owned_buffers(backend, oracle):
    m, in_f, out_f = 3, 1024, 200
    w = synth.weight(Q4K, out_f, in_f, seed=11)
    x = synth.normal(12, (m, in_f))
    wb, xb, yb = backend.from_numpy(w, infr_b200.USAGE_WEIGHTS), backend.from_numpy(x), backend.alloc(m * out_f * 4)
    backend.linear(Q4K, wb, xb, yb, m, in_f, out_f)
    want = backend.download(yb, np.float32).reshape(m, out_f)
    # the same memory through non-owning handles
    y2 = backend.alloc(m * out_f * 4)
    ww = backend.wrap(wb.device_ptr(), w.nbytes, infr_b200.USAGE_WEIGHTS)
    xw = backend.wrap(xb.device_ptr(), x.nbytes, infr_b200.USAGE_ACTIVATIONS)
    yw = backend.wrap(y2.device_ptr(), m * out_f * 4, infr_b200.USAGE_ACTIVATIONS)
    assert ww.len_bytes() == w.nbytes and ww.device_ptr() == wb.device_ptr()
    backend.linear(Q4K, ww, xw, yw, m, in_f, out_f)
    got = backend.download(y2, np.float32).reshape(m, out_f)
    np.testing.assert_array_equal(got, want)
    assert fx.rel_l2(got, oracle.linear(Q4K, w, x, m, in_f, out_f)) < 1e-3
    # dropping the handles leaves the memory alone
    for h in (ww, xw, yw):
        h.close()
    backend.linear(Q4K, wb, xb, yb, m, in_f, out_f)
    np.testing.assert_array_equal(backend.download(yb, np.float32).reshape(m, out_f), want)


def test_wrap_rejects_null_empty_and_misaligned(backend):
    b = backend.alloc(256)
    for ptr, n in ((0, 64), (b.device_ptr(), 0), (b.device_ptr() + 4, 64)):
        with pytest.raises(infr_b200.BackendError) as e:
            backend.wrap(ptr, n)
        assert e.value.code == infr_b200.E_INVALID


def test_stream_is_usable_from_torch(backend):
    torch = pytest.importorskip("torch")
    s = backend.stream()
    assert s != 0  # the context owns a stream of its own
    ext = torch.cuda.ExternalStream(s)
    m, in_f, out_f = 1, 512, 64
    w = synth.weight(Q4K, out_f, in_f, seed=21)
    wb = backend.from_numpy(w, infr_b200.USAGE_WEIGHTS)
    with torch.cuda.stream(ext):
        x = torch.ones(in_f, device="cuda")
        y = torch.zeros(out_f, device="cuda")
        ext.synchronize()
        xw, yw = backend.wrap(x.data_ptr(), in_f * 4, infr_b200.USAGE_ACTIVATIONS), backend.wrap(y.data_ptr(), out_f * 4, infr_b200.USAGE_ACTIVATIONS)
        backend.linear(Q4K, wb, xw, yw, m, in_f, out_f)
        y2 = y * 2.0  # a torch kernel ordered after the Linear on the shared stream
        ext.synchronize()
    want = backend.run_linear(Q4K, w, np.ones((1, in_f), np.float32), m, in_f, out_f)
    np.testing.assert_allclose(y2.cpu().numpy(), 2.0 * want[0], rtol=0, atol=0)


def test_small_uploads_do_not_alias_when_the_source_is_reused(backend):
    """upload() of a small buffer returns before the copy has run (it goes through a ring of pinned slots); the
    caller's source may be overwritten at once, as the trait's borrowed slice allows, and more uploads than the
    ring has slots must still land with their own bytes."""
    n_buf, n = 40, 4096
    host = backend.host_array((n,), np.float32)
    bufs = [backend.alloc(n * 4) for _ in range(n_buf)]
    for i, b in enumerate(bufs):
        host[:] = np.float32(i) + np.arange(n, dtype=np.float32) / n
        backend.upload_raw(b, host.ctypes.data, n * 4)
        host[:] = -1.0  # reuse of the source right after the call
    for i, b in enumerate(bufs):
        want = np.float32(i) + np.arange(n, dtype=np.float32) / n
        np.testing.assert_array_equal(backend.download(b, np.float32), want)
    # a size that spans the small / large boundary on both sides
    for nbytes in (64 << 10, (64 << 10) + 256):
        src = np.arange(nbytes, dtype=np.uint8)
        big = backend.alloc(nbytes)
        backend.upload(big, src)
        np.testing.assert_array_equal(backend.download(big, np.uint8), src)
