"""The device-side failure path, exercised without faulting or hanging anything: a kernel waits on a barrier that
nothing completes; the wait is bounded (here 50 ms), records the failure, the kernel ends normally, the host reads
MD_ERR_TIMEOUT at the next synchronisation and the context keeps working."""
import numpy as np
import pytest

from conftest import assert_close_ref, f16_normal

pytestmark = pytest.mark.gpu


def test_bounded_wait_reports_timeout_and_context_stays_usable(ctx, pkg, oracle):
    ctx.sync()                                   # clean state
    ctx.selftest_bounded_wait(50)
    with pytest.raises(pkg.MdError) as e:
        ctx.sync()
    assert e.value.status == 9                   # MD_ERR_TIMEOUT
    assert "site 99" in str(e.value)
    ctx.sync()                                   # the error was consumed: the context is clean again
    rng = np.random.default_rng(1)
    a, b = f16_normal(rng, (4, 256)), f16_normal(rng, (128, 256), 0.05)
    assert_close_ref(ctx.hgemm_nt(a, b, 4, 128, 256), oracle.hgemm_nt(a, b), "GEMV after a reported timeout")


def test_timeout_is_reported_by_a_call_with_host_output(ctx, pkg):
    ctx.sync()
    ctx.selftest_bounded_wait(20)
    rng = np.random.default_rng(2)
    a, b = f16_normal(rng, (1, 64)), f16_normal(rng, (16, 64))
    with pytest.raises(pkg.MdError) as e:        # host output: the call synchronises and sees the flag
        ctx.hgemm_nt(a, b, 1, 16, 64)
    assert e.value.status == 9
    ctx.sync()


def test_selftest_rejects_unbounded_limits(ctx, pkg):
    with pytest.raises(pkg.MdError):
        ctx.selftest_bounded_wait(0)
    with pytest.raises(pkg.MdError):
        ctx.selftest_bounded_wait(60000)
