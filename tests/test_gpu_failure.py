"""GPU: failure paths in the forms that never fault, trap or hang a device.

A bounded wait is made to run out on a barrier that nothing completes: the kernel returns, the status word carries
EB_DEV_WAIT_TIMEOUT, and the context keeps working.  (A device-side fault injector is deliberately not part of the
library; rank failures are injected on the host, see tests/test_failure_gloo.py.)"""
import ctypes as C

import numpy as np
import pytest

from tests.helpers import AttnCase, assert_close_bf16

pytestmark = pytest.mark.gpu


def test_a_bounded_wait_runs_out_and_the_context_stays_usable(gpu):
    import eidola_b200 as eb
    from eidola_b200 import capi
    polls = C.c_uint32(0)
    capi.call("eb_selftest_wait_expires", C.c_uint32(4096), C.byref(polls))
    assert polls.value == 4096                      # the wait gave up exactly at its limit ...
    st = eb.status_read()
    assert st & 0x1000 and not st & 0x2000          # ... and said so; reading clears the word
    assert eb.status_read() == 0
    # the same context still computes correctly afterwards
    case = AttnCase([7, 250, 1500], [1, 1, 1], 8, seed=21, sm_count=gpu["sm_count"])
    got, _ = case.run(0, 16)
    assert_close_bf16(got, case.oracle(0), what="attention after a timed-out wait")
    assert eb.status_read() == 0


def test_wait_limit_is_a_runtime_setting(gpu):
    from eidola_b200 import capi
    cur = C.c_uint32(0)
    capi.call("eb_wait_limit_get", C.byref(cur))
    assert cur.value >= 1
    capi.call("eb_wait_limit_set", C.c_uint32(1 << 20))
    got = C.c_uint32(0)
    capi.call("eb_wait_limit_get", C.byref(got))
    assert got.value == 1 << 20
    assert capi.call_rc("eb_wait_limit_set", C.c_uint32(0)) == -1  # refused, nothing changed
    # kernels launched now carry the new limit and still finish long before it
    case = AttnCase([33, 900], [1, 1], 8, seed=22, sm_count=gpu["sm_count"])
    got_out, _ = case.run(0, 8)
    assert_close_bf16(got_out, case.oracle(0), what="attention with a 2^20-poll limit")
    capi.call("eb_wait_limit_set", cur)
