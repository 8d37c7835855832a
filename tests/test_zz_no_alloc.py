"""cs1_gdn_prefill_static: the delta rule for callers that cannot allocate device memory.

Some users of the library cannot give cs1_gdn_prefill a workspace: they run inside a process
whose device memory belongs to someone else, or on a path where cudaMalloc is not allowed
because it stalls the whole GPU. The static entry point keeps its workspace in a fixed 64 MiB
array inside the library instead. This file checks, through the C ABI, that it returns
exactly what the workspace-taking entry point returns - twice in a row with different
inputs, because the array keeps the previous call's contents - and that it refuses windows
that do not fit. It is collected last so that a run that stops at the first failure has
already run every other test; it does not depend on any of them.
"""
import numpy as np
import pytest

from helpers import gdn_inputs
from system1_omni_b200 import lib as L

pytestmark = pytest.mark.gpu
STATIC_BYTES = 64 << 20
ERR_STATIC_SCRATCH = 2003


def with_workspace(cs1, stream, q, k, v, g, beta, t, h, hk):
    qd, kd, vd, gd, bd = (L.to_device(a, stream) for a in (q, k, v, g, beta))
    o = L.DeviceBuffer(t * h * 128 * 2)
    ws = L.DeviceBuffer(cs1.cs1_gdn_workspace_floats(t, h) * 4)
    L.check(cs1.cs1_gdn_prefill(qd.at(), kd.at(), vd.at(), gd.at(), bd.at(), o.at(), ws.at(), t, h, hk, 128 ** -0.5,
                                stream.handle), "gdn prefill")
    return L.from_device(o, (t, h, 128), np.uint16, stream)


def without_allocation(cs1, stream, q, k, v, g, beta, t, h, hk):
    qd, kd, vd, gd, bd = (L.to_device(a, stream) for a in (q, k, v, g, beta))
    o = L.DeviceBuffer(t * h * 128 * 2)
    L.check(cs1.cs1_gdn_prefill_static(qd.at(), kd.at(), vd.at(), gd.at(), bd.at(), o.at(), t, h, hk, 128 ** -0.5,
                                       stream.handle), "gdn prefill static")
    return L.from_device(o, (t, h, 128), np.uint16, stream)


def test_static_scratch_matches_the_workspace_entry_point_twice_in_a_row(cs1, stream):
    # two calls back to back on one stream: a large window, then a shorter one with other
    # values, so that anything stale from the first call would show in the second
    cases = [(1024, 32, 16, 0.3, 1.0), (200, 4, 2, 1.0, 1.0)]
    for t, h, hk, decay, amp in cases:
        assert cs1.cs1_gdn_workspace_floats(t, h) * 4 <= STATIC_BYTES
        q, k, v, g, beta = gdn_inputs(t, h, hk, decay, amp)
        got = without_allocation(cs1, stream, q, k, v, g, beta, t, h, hk)
        want = with_workspace(cs1, stream, q, k, v, g, beta, t, h, hk)
        assert np.array_equal(got, want), f"static scratch changed the result at T={t}, H={h}"
    # and once more on the first shape: identical to its first result
    t, h, hk, decay, amp = cases[0]
    q, k, v, g, beta = gdn_inputs(t, h, hk, decay, amp)
    again = without_allocation(cs1, stream, q, k, v, g, beta, t, h, hk)
    assert np.array_equal(again, with_workspace(cs1, stream, q, k, v, g, beta, t, h, hk))


def test_static_scratch_limits(cs1, stream):
    st = stream.handle
    # a window whose workspace exceeds the fixed array is refused before anything is launched
    assert cs1.cs1_gdn_workspace_floats(16384, 48) * 4 > STATIC_BYTES
    assert cs1.cs1_gdn_prefill_static(None, None, None, None, None, None, 16384, 48, 16, 1.0, st) == ERR_STATIC_SCRATCH
    assert b"fixed scratch" in cs1.cs1_error_string(ERR_STATIC_SCRATCH)
    # the largest windows that fit, as documented: 1792 tokens at 32 heads, 1152 at 48, 3584 at 16
    for t, h in [(1792, 32), (1152, 48), (3584, 16)]:
        assert cs1.cs1_gdn_workspace_floats(t, h) * 4 <= STATIC_BYTES
        assert cs1.cs1_gdn_workspace_floats(t + 64, h) * 4 > STATIC_BYTES
    # no tokens is a no-op; bad head grouping is an argument error, as for the other entry points
    assert cs1.cs1_gdn_prefill_static(None, None, None, None, None, None, 0, 4, 2, 1.0, st) == 0
    assert cs1.cs1_gdn_prefill_static(None, None, None, None, None, None, 5, 4, 3, 1.0, st) == 1
