"""A bounded wait that runs out, on a live GPU, without a fault.

The kernels never spin for ever: every wait on a barrier carries a time limit, after which the role that waited
records a code in a status word, the block winds down and the kernel returns.  `disc_b200_selftest_wait_expiry`
launches one warp that waits with that same code on a barrier nobody will arrive on (nothing is in flight), with the
limit set to a millisecond.  The test checks that the kernel came back after about that long, that
`disc_b200_kernel_status()` names the wait and is clear afterwards, and that the next ordinary launch is correct."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_reports_and_returns():
    from bladedisc_b200 import lib as L
    from bladedisc_b200 import ops
    from oracle import c
    lib = L.load()
    assert ops.kernel_status() == 0
    waited = ctypes.c_int64(0)
    stream = torch.cuda.current_stream().cuda_stream
    L.check(lib.disc_b200_selftest_wait_expiry(1_000_000, ctypes.byref(waited), stream))   # 1 ms
    assert 1_000_000 <= waited.value < 50_000_000, f"the wait lasted {waited.value} ns"
    assert lib.disc_b200_kernel_status() == 9        # the self-test's code
    assert lib.disc_b200_kernel_status() == 0        # read once, then clear
    # the context is intact: an ordinary launch right after is correct
    rng = np.random.default_rng(1)
    a = rng.integers(-127, 128, (300, 256), dtype=np.int8)
    w = rng.integers(-127, 128, (192, 256), dtype=np.int8)
    got = ops.qgemm(torch.from_numpy(a).cuda(), torch.from_numpy(w).cuda(), out_dtype=torch.int32).cpu().numpy()
    assert (got == c.qgemm_acc(a, w)).all()
    assert ops.kernel_status() == 0


def test_the_self_test_refuses_long_limits():
    from bladedisc_b200 import lib as L
    lib = L.load()
    waited = ctypes.c_int64(0)
    assert lib.disc_b200_selftest_wait_expiry(10**10, ctypes.byref(waited), None) != 0
    assert b"100 ms" in lib.disc_b200_last_error_string()
