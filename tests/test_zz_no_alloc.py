"""GPU: the attention entry point that allocates nothing, against the ordinary one.

Collected last (file name) so that a run that stops at the first failure has already run every other test.
The entry point exists for hosts that cannot call cudaMalloc at the point where they need attention -- all device
memory already belongs to their own pool, or they run inside another runtime's arena, or the calling thread must
not take the allocator's lock -- so its split-K scratch is a pair of arrays built into the library.  Both entry
points launch the same kernels on the same plan, so their outputs must be identical bit for bit; two calls in a row
(the second on another batch and layer type) check that what the first call left in the shared scratch is harmless.
"""
import numpy as np
import pytest

from tests.helpers import AttnCase

pytestmark = pytest.mark.gpu


def _run_both(case, window, chunk):
    from eidola_b200 import capi
    from eidola_b200.capi import DeviceBuffer
    from eidola_b200.host import attn_paged_sink_static
    launch, plan = case.launch(window, chunk)
    case.d_out.zero()
    launch.run()
    capi.call("eb_device_sync")
    want = case.d_out.to_array(np.uint16, (case.T, case.n_q * 64))
    d_status = DeviceBuffer.from_array(np.zeros(1, np.int32))
    launch.args.d_part_acc = None  # the static variant must not need them
    launch.args.d_part_ml = None
    case.d_out.zero()
    capi.call("eb_device_sync")
    free_before, _ = capi.mem_info()
    attn_paged_sink_static(launch.args, d_status.ptr)
    capi.call("eb_device_sync")
    free_after, _ = capi.mem_info()
    got = case.d_out.to_array(np.uint16, (case.T, case.n_q * 64))
    assert d_status.to_array(np.int32, 1)[0] == 0
    assert plan["n_parts"] > len(case.packed["slots"]) or window  # split-K really used the scratch
    assert np.array_equal(got, want)
    return plan, free_before, free_after


def test_static_scratch_attention_matches_on_two_calls_in_a_row(gpu):
    import eidola_b200 as eb
    from eidola_b200.host import attn_paged_sink_static
    a = AttnCase([7, 33, 128, 250, 1000, 2049, 5000], [1, 1, 1, 1, 1, 1, 1], 8, seed=11, sm_count=gpu["sm_count"])
    _run_both(a, window=0, chunk=8)  # the first call on the device also resolves the scratch addresses
    b = AttnCase([300, 45, 1100, 16, 4000], [5, 2, 1, 1, 3], 2, seed=12, sm_count=gpu["sm_count"], group=4)
    _, f0, f1 = _run_both(b, window=0, chunk=5)
    assert f0 == f1, "the second call changed the device's free memory: something was allocated"
    _, f0, f1 = _run_both(b, window=128, chunk=0)
    assert f0 == f1
    # beyond the built-in scratch: refused with a clear error, nothing launched
    big = AttnCase([40000], [1], 8, seed=13, sm_count=gpu["sm_count"])
    launch, plan = big.launch(0, 1)  # one page per item: 2500 partial slots x 64 heads > 65536 rows
    assert plan["n_parts"] * 64 > 65536
    with pytest.raises(eb.EbError) as e:
        attn_paged_sink_static(launch.args)
    assert e.value.code == -3 and "built-in scratch" in str(e.value)
    assert eb.status_read() == 0


def test_static_scratch_status_without_a_caller_word(gpu):
    """d_status = NULL: the EB_DEV_* bits land in the library's own word, which both readers report and clear."""
    import eidola_b200 as eb
    from eidola_b200 import capi
    from eidola_b200.capi import DeviceBuffer
    from eidola_b200.host import attn_paged_sink_static
    case = AttnCase([40, 700], [1, 1], 8, seed=14, sm_count=gpu["sm_count"])
    bad = case.bt.copy()
    bad[0, 1] = case.num_pages + 7  # out of range: the kernel skips the page and raises the flag, it never dereferences it
    case.d_bt = DeviceBuffer.from_array(bad)
    for reader in (capi.static_status_read, eb.status_read):
        launch, _ = case.launch(0, 8)
        attn_paged_sink_static(launch.args, None)
        capi.call("eb_device_sync")
        assert reader() & 0x2000
        assert capi.static_status_read() == 0 and eb.status_read() == 0


@pytest.mark.parametrize("q_len", [1, 5])
def test_static_scratch_refuses_a_partial_slot_outside_the_plan(gpu, q_len):
    """A plan whose items name a partial slot >= n_parts (a stale plan) is skipped and flagged, not followed past the
    built-in arrays: the rows of the other sequences are still right, and the flagged sequence's output is untouched.
    q_len 1 runs the decode kernel, q_len 5 the tcgen05 verify kernel."""
    from eidola_b200 import capi
    from eidola_b200.capi import DeviceBuffer
    from eidola_b200.host import attn_paged_sink_static
    case = AttnCase([2000, 900], [q_len, q_len], 8, seed=15, sm_count=gpu["sm_count"])
    launch, plan = case.launch(0, 16)
    case.d_out.zero()
    launch.run()
    capi.call("eb_device_sync")
    want = case.d_out.to_array(np.uint16, (case.T, case.n_q * 64))
    items = np.array(plan["items"], np.int32).reshape(-1, 4).copy()
    victim = int(np.nonzero(items[:, 0] == 0)[0][0])
    items[victim, 3] = plan["n_parts"] + 1000  # far beyond the partial slots of this launch
    launch.bufs["items"] = DeviceBuffer.from_array(items)
    launch.args.d_items = launch.bufs["items"].ptr
    d_status = DeviceBuffer.from_array(np.zeros(1, np.int32))
    case.d_out.zero()
    attn_paged_sink_static(launch.args, d_status.ptr)
    capi.call("eb_device_sync")
    assert d_status.to_array(np.int32, 1)[0] & 0x2000
    got = case.d_out.to_array(np.uint16, (case.T, case.n_q * 64))
    assert np.array_equal(got[q_len:], want[q_len:])  # the sequence whose plan was intact
