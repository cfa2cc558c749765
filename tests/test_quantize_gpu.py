"""On-GPU activation quantiser vs the CPU restatement: every output bit-exact."""
import numpy as np
import pytest

import fixtures as fx
from infr_b200 import synth

pytestmark = pytest.mark.gpu


def _inputs(rows, k, seed):
    x = synth.normal(seed, (rows, k))
    x[0, :32] = 0.0                      # an all-zero block: d = 0 -> id = 0 -> codes 0
    if k >= 512:
        x[-1, 256:512] *= 1e-30          # denormal-scale block
    x[rows // 2, k // 2] = 1234.5        # an outlier that pins amax
    x[0, 40] = 0.5 * np.abs(x[0, 32:64]).max() / 127 * 3  # lands near a .5 rounding boundary
    if k > 70:
        x[0, 70] = np.nan                # a NaN element: its code is 0 (Rust's `as i8`), the block's amax ignores it
    if k >= 512:
        x[0, 300] = np.inf               # an infinite element: d = inf -> id = 0 -> every code of the block 0
    if k >= 768:
        x[-1, 512:768] *= 1e-38          # amax / 127 is so small that its reciprocal is infinite: codes are +-127 or 0
    return x


@pytest.mark.parametrize("rows,k", [(1, 256), (1, 4096), (5, 768), (8, 14336), (33, 2048), (512, 4096)])
def test_quantize_q8_256_bit_exact(backend, oracle, rows, k):
    x = _inputs(rows, k, 1000 + rows + k)
    xb = backend.from_numpy(x)
    qs = backend.alloc(rows * k)
    d = backend.alloc(rows * (k // 256) * 4)
    s32 = backend.alloc(rows * (k // 32) * 4)
    s16 = backend.alloc(rows * (k // 16) * 4)
    backend.quantize_q8(256, xb, rows, k, qs, d, s32, s16)
    g_qs = backend.download(qs, np.int8).reshape(rows, k)
    g_d = backend.download(d, np.float32).reshape(rows, -1)
    g_s = backend.download(s32, np.int32).reshape(rows, -1)
    g_s16 = backend.download(s16, np.int32).reshape(rows, -1)
    for r in range(rows):
        o_qs, o_d, o_s, o_s16 = oracle.quantize_q8(x[r])
        np.testing.assert_array_equal(g_qs[r], o_qs)
        np.testing.assert_array_equal(g_d[r].view(np.uint32), o_d.view(np.uint32))
        np.testing.assert_array_equal(g_s[r], o_s)
        np.testing.assert_array_equal(g_s16[r], o_s16)


@pytest.mark.parametrize("rows,k", [(1, 64), (1, 704), (3, 14336), (4, 4096), (256, 768)])
def test_quantize_q8_32_and_q8_1_bit_exact(backend, oracle, rows, k):
    x = _inputs(rows, k, 2000 + rows + k)
    xb = backend.from_numpy(x)
    qs = backend.alloc(rows * k)
    d = backend.alloc(rows * (k // 32) * 4)
    s32 = backend.alloc(rows * (k // 32) * 4)
    backend.quantize_q8(32, xb, rows, k, qs, d, s32)
    g_qs = backend.download(qs, np.int8).reshape(rows, k)
    g_d = backend.download(d, np.float32).reshape(rows, -1)
    g_s = backend.download(s32, np.int32).reshape(rows, -1)
    qs1 = backend.alloc(rows * k)
    dact = backend.alloc(rows * (k // 32) * 2)
    sact = backend.alloc(rows * (k // 32) * 2)
    backend.quantize_q8_1(xb, rows, k, qs1, dact, sact)
    g_qs1 = backend.download(qs1, np.int8).reshape(rows, k)
    g_da = backend.download(dact, np.uint16).reshape(rows, -1)
    g_sa = backend.download(sact, np.uint16).reshape(rows, -1)
    for r in range(rows):
        o_qs, o_d, o_s = oracle.quantize_q8_32(x[r])
        np.testing.assert_array_equal(g_qs[r], o_qs)
        np.testing.assert_array_equal(g_d[r].view(np.uint32), o_d.view(np.uint32))
        np.testing.assert_array_equal(g_s[r], o_s)
        o_qs1, o_da, o_sa = oracle.quantize_q8_1(x[r])
        np.testing.assert_array_equal(g_qs1[r], o_qs1)
        np.testing.assert_array_equal(g_da[r], o_da)
        # d * sum is inf * 0 = NaN for the block that holds the infinite element: a NaN on both sides (the payload
        # and sign of a generated NaN are the hardware's), every other value bit for bit
        nan_g, nan_o = np.isnan(g_sa[r].view(np.float16)), np.isnan(o_sa.view(np.float16))
        np.testing.assert_array_equal(nan_g, nan_o)
        np.testing.assert_array_equal(g_sa[r][~nan_g], o_sa[~nan_o])


def test_quantize_rejects_bad_shapes(backend):
    import infr_b200

    xb = backend.alloc(1024 * 4)
    qs = backend.alloc(1024)
    d = backend.alloc(64)
    s = backend.alloc(256)
    with pytest.raises(infr_b200.BackendError) as ei:
        backend.quantize_q8(256, xb, 1, 1000, qs, d, s)
    assert ei.value.code == infr_b200.E_INVALID
    with pytest.raises(infr_b200.BackendError):
        backend.quantize_q8(64, xb, 1, 1024, qs, d, s)
    with pytest.raises(infr_b200.BackendError):   # output too small
        backend.quantize_q8(256, xb, 2, 1024, qs, d, s)
    # the quantiser is idempotent on re-run (no hidden state): run twice, same bits
    x = synth.normal(7, (1, 1024))
    backend.upload(xb, x)
    backend.quantize_q8(256, xb, 1, 1024, qs, d, s)
    a = backend.download(qs, np.int8).copy()
    backend.quantize_q8(256, xb, 1, 1024, qs, d, s)
    np.testing.assert_array_equal(a, backend.download(qs, np.int8))
