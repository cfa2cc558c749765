"""The dense int8 tensor-core peak microbenchmark: it runs, its accumulator check passes (the entry point returns an
error otherwise), and the rate it reports is that of a B200's tensor cores, not of something that skipped the work."""
import pytest

pytestmark = pytest.mark.gpu


def test_int8_peak_is_plausible_and_checked(backend):
    ms, ops = backend.tensor_peak_i8(n_batches=8, launches=4)
    sms = backend.capabilities().sm_count
    assert ops == 2.0 * 128 * 256 * 32 * 64 * 8 * 2 * sms * 4
    tops = ops / (ms * 1e-3) / 1e12
    # the datasheet's dense int8 figure is 4.5 POPS; anything far above it would mean the loop did not run
    assert 500.0 < tops < 5500.0, tops


def test_int8_peak_argument_checks(backend):
    import infr_b200

    for nb, nl in ((0, 1), (5000, 1), (1, 0)):
        with pytest.raises(infr_b200.BackendError) as e:
            backend.tensor_peak_i8(n_batches=nb, launches=nl)
        assert e.value.code == infr_b200.E_INVALID
