"""The failure-detection path of the kernels, exercised without faulting anything: every device-side
wait is bounded, and a wait that runs out records a status bit, raises the CTA's abort flag and lets
the kernel return normally.  Here one such wait is made to run out on purpose (a barrier nobody
arrives at, 1 ms budget) and the host-side reporting is checked, together with the rule for
non-finite inputs that the header states."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(x, cuda):
    import torch

    return torch.from_numpy(np.ascontiguousarray(x)).to(cuda)


def test_a_wait_that_runs_out_is_reported_once_and_the_context_stays_usable(pkg, orc, cuda):
    import torch

    g = orc.Rng(5)
    a, b = g.randn((200, 300)), g.randn((300, 150))
    A, B = dev(a, cuda), dev(b, cuda)
    before = pkg.matmul(A, B)
    pkg.status()  # clean so far
    wrongly_completed, abort_flag = pkg.selftest_timeout(1000)
    assert wrongly_completed == 0, "a wait on a barrier nobody arrives at reported completion"
    assert abort_flag == 1, "the abort flag that makes the other roles leave was not raised"
    with pytest.raises(pkg.B200Error) as err:
        pkg.status()
    assert err.value.code == -5  # B200_ETIMEDOUT
    pkg.status()  # reported once, then clear
    after = pkg.matmul(A, B)
    pkg.status()
    assert torch.equal(before, after)
    assert orc.scaled_error(after.cpu().numpy(), orc.matmul(a, b)) <= orc.parity_tolerance(300)


def test_selftest_rejects_unbounded_budgets(pkg, cuda):
    for bad in (0, 100001):
        with pytest.raises(pkg.B200Error) as err:
            pkg.selftest_timeout(bad)
        assert err.value.code == -1


def test_zeros_in_a_behave_like_the_reference_skip_for_finite_inputs(pkg, orc, cuda):
    """The reference skips terms with a == 0 (src/tensor_ops.cpp:555); with finite inputs that
    changes nothing, so whole zero rows, zero columns of A and scattered zeros must match."""
    g = orc.Rng(6)
    a, b = g.randn((130, 70)), g.randn((70, 90))
    a[3] = 0.0
    a[:, 11] = 0.0
    a[::7, ::5] = 0.0
    got = pkg.matmul(dev(a, cuda), dev(b, cuda))
    pkg.status()
    got = got.cpu().numpy()
    want = orc.matmul(a, b)
    assert orc.scaled_error(got, want) <= 1e-5
    assert not got[3].any() and not np.signbit(got[3]).any()  # an all-zero row gives +0, as in the reference


def test_non_finite_inputs_differ_from_the_reference_as_documented(pkg, orc, cuda):
    """include/b200_gemm.h: finite inputs only.  An infinite B value met by a zero A value is
    skipped by the reference (that output stays finite) and is not finite here; the other outputs of
    the column are +-inf there and NaN or +-inf here; columns that do not touch the value are
    unaffected."""
    g = orc.Rng(7)
    a, b = g.randn((64, 40)), g.randn((40, 48))
    a[0, 5] = 0.0
    b[5, 9] = np.inf
    want = orc.matmul(a, b)
    assert np.isfinite(want[0]).all()            # the reference never formed 0 * inf
    assert np.isinf(want[1:, 9]).all()           # the other rows hold +-inf there
    got = pkg.matmul(dev(a, cuda), dev(b, cuda))
    pkg.status()
    got = got.cpu().numpy()
    assert not np.isfinite(got[:, 9]).any()      # documented: NaN or +-inf, the skipped term included
    assert np.isnan(got[0, 9])                   # 0 * inf was formed
    cols = np.arange(48) != 9
    assert orc.scaled_error(got[:, cols], want[:, cols]) <= 1e-5
