"""The allocation-free GEMV entry point against the regular one.

Who needs it: a caller that is handed device pointers from somebody else's pool, or that has promised
not to touch the CUDA allocator once it is running, cannot use the regular entry points (their
quantised activations live in a buffer the context grows on demand).  infr_cuda_gemv_noalloc keeps that
scratch in an array built into the library instead.  This test drives it through the C ABI with raw
device pointers, twice in a row on different inputs (the second call reuses the scratch the first one
filled), and expects the same numbers as infr_cuda_gemv within the tolerance of the GEMV tests.
"""
import ctypes as C

import numpy as np
import pytest

import fixtures as fx
import infr_b200
from fixtures import Q2_0, Q4K, Q6K
from infr_b200 import synth

pytestmark = pytest.mark.gpu

TIGHT_REL_L2 = 2e-5


def _sync_device():
    import torch

    torch.cuda.synchronize()


def _noalloc(lib, dt, wb, xb, yb, m, in_f, out_f, w_skew=0, x_skew=0, y_skew=0):
    err = C.create_string_buffer(256)
    rc = lib.infr_cuda_gemv_noalloc(dt, wb.device_ptr() + w_skew, xb.device_ptr() + x_skew, yb.device_ptr() + y_skew, m, in_f, out_f,
                                    None, err, 256)
    return rc, err.value.decode()


# the last case is the documented maximum (8 rows of 16384 activations): the largest staging the entry point accepts
@pytest.mark.parametrize("dt,in_f,out_f", [(Q6K, 4096, 1536), (Q2_0, 14336, 512), (Q4K, 2048, 768), (Q4K, 16384, 64)])
def test_noalloc_matches_regular_entry_point_twice(backend, dt, in_f, out_f):
    lib = infr_b200.load_library()
    w = synth.weight(dt, out_f, in_f, seed=41 + dt)
    wb = backend.from_numpy(w, infr_b200.USAGE_WEIGHTS)
    for call, m in enumerate((8, 3)):           # second call: fewer rows, scratch still holds the first call's
        x = synth.normal(60 + call, (m, in_f)) * np.float32(1 + call)
        xb = backend.from_numpy(x)
        y_ref = backend.alloc(m * out_f * 4)
        y_new = backend.alloc(m * out_f * 4)
        backend.gemv(dt, wb, xb, y_ref, m, in_f, out_f, infr_b200.ACT_INT8)
        backend.sync()
        rc, msg = _noalloc(lib, dt, wb, xb, y_new, m, in_f, out_f)
        assert rc == 0, msg
        _sync_device()
        want = backend.download(y_ref, np.float32)
        got = backend.download(y_new, np.float32)
        assert np.abs(want).max() > 1e-3
        assert fx.rel_l2(got, want) < TIGHT_REL_L2


def test_noalloc_rejects_sizes_beyond_its_scratch(backend):
    lib = infr_b200.load_library()
    b = backend.alloc(1 << 20)
    rc, msg = _noalloc(lib, Q4K, b, b, b, 9, 4096, 16)          # m > 8
    assert rc == infr_b200.E_INVALID and "at most" in msg
    rc, msg = _noalloc(lib, Q4K, b, b, b, 1, 16384 + 256, 16)   # in_f > 16384
    assert rc == infr_b200.E_INVALID and "at most" in msg
    rc, msg = _noalloc(lib, 5, b, b, b, 1, 4096, 16)            # a dtype this library does not run
    assert rc == infr_b200.E_UNSUPPORTED
    # pointers at odd offsets of a pool are refused on the host (nothing is launched): x needs 16 bytes, y 4,
    # w 16 for Q4_K and 2 for the other formats
    for kw in (dict(x_skew=4), dict(y_skew=2), dict(w_skew=8)):
        rc, msg = _noalloc(lib, Q4K, b, b, b, 1, 4096, 16, **kw)
        assert rc == infr_b200.E_INVALID and "misaligned" in msg, kw
    rc, msg = _noalloc(lib, Q6K, b, b, b, 1, 4096, 16, w_skew=1)
    assert rc == infr_b200.E_INVALID and "misaligned" in msg
    err = C.create_string_buffer(64)
    assert lib.infr_cuda_gemv_noalloc(Q4K, None, None, None, 1, 4096, 16, None, err, 64) == infr_b200.E_INVALID
