"""Bounded device-side waits: a wait that can never be satisfied runs out, the kernel still
finishes, the failure is reported to the caller, and the context stays usable.  The failure
is made by a test option of the library that drops ONE carry hand-over per launch (nothing
faults, traps or hangs).  Also: the launch epoch that tags carry words may wrap."""
import ctypes

import pytest
import torch

from helpers import real_inputs, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

ROWS, T = 7200, 16000          # chained stream plan: more than four rows per warp, several segments per row


@pytest.fixture
def chained_case(cuda_device):
    from accelerated_scan import _native

    pl = _native.plan(ROWS, T, _native.F32, _native.KIND_FORWARD)
    assert pl["kernel"] == 0 and pl["segs_per_row"] > 1 and pl["dynamic"] == 1
    gates, tokens, _ = real_inputs(2, (1, ROWS, T), grad=False)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    g, x = gates.to(cuda_device), tokens.to(cuda_device)
    _native.check_status(cuda_device)                     # clean before
    yield g, x, want
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 0)
    _native.set_debug(False)


def test_expired_wait_is_reported_and_context_survives(cuda_device, chained_case):
    from accelerated_scan import _native

    g, x, want = chained_case
    out = torch.empty_like(x)
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 1)
    _native.forward(g, x, out)                            # row 0 loses the state between two segments
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        _native.check_status(cuda_device)
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 0)
    # the status word was cleared by the check, the workspace rearmed itself: a normal call is right
    _native.forward(g, x, out)
    _native.check_status(cuda_device)
    assert rel_err(to_np(out), want) <= 1e-5


def test_debug_mode_raises_from_the_scan_call_itself(cuda_device, chained_case):
    """With the check mode on (ASCAN_CHECK=1 or set_debug) the drop-in API raises where the
    reference would (a RuntimeError out of the call, warp.cuh:396-401)."""
    from accelerated_scan import _native
    import accelerated_scan.warp as warp

    g, x, want = chained_case
    _native.set_debug(True)
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 1)
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        warp.scan_forward(g.view(1, ROWS, T), x.view(1, ROWS, T))
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 0)
    out = warp.scan_forward(g.view(1, ROWS, T), x.view(1, ROWS, T))
    assert rel_err(to_np(out), want) <= 1e-5


def test_failure_surfaces_at_the_next_call_without_debug_mode(cuda_device, chained_case):
    """Without the check mode nothing synchronises; the kernel leaves its status in pinned
    host memory as well, and the next call on that stream raises before it launches."""
    from accelerated_scan import _native

    g, x, want = chained_case
    out = torch.empty_like(x)
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 1)
    _native.forward(g, x, out)
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 0)
    torch.cuda.synchronize(cuda_device)                   # the failed launch has finished
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        _native.forward(g, x, out)
    _native.check_status(cuda_device)                     # reported once: both copies of the status are clear
    _native.forward(g, x, out)
    _native.check_status(cuda_device)
    assert rel_err(to_np(out), want) <= 1e-5


def test_no_alloc_entry_point_keeps_its_timeout_until_asked(cuda_device, chained_case):
    from accelerated_scan import _native

    g, x, want = chained_case
    lib = _native.lib
    out = torch.empty_like(x)
    stream = torch.cuda.current_stream(cuda_device).cuda_stream
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    assert lib.ascan_check_no_alloc(stream) == 0
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 1)
    assert lib.ascan_forward_no_alloc(p(g), p(x), p(out), ROWS, T, _native.F32, 0, stream) == 0
    _native.set_option(_native.OPT_TEST_DROP_CARRY, 0)
    # a second call does not erase the first call's failure
    assert lib.ascan_forward_no_alloc(p(g), p(x), p(out), ROWS, T, _native.F32, 0, stream) == 0
    assert lib.ascan_check_no_alloc(stream) == 4
    assert lib.ascan_check_no_alloc(stream) == 0
    assert rel_err(to_np(out), want) <= 1e-5


def test_launch_epoch_may_wrap(cuda_device):
    """Carry words are tagged with the launch epoch; the launch that wraps the epoch wipes
    the records.  With a 2-bit epoch, twelve launches of alternating shapes on one workspace
    cross the wrap three times and stay correct."""
    from accelerated_scan import _native

    cases = []
    for seed, (rows, t) in enumerate([(7200, 16000), (7300, 14000)]):
        assert _native.plan(rows, t, _native.F32, _native.KIND_FORWARD)["segs_per_row"] > 1
        gates, tokens, _ = real_inputs(40 + seed, (1, rows, t), grad=False)
        cases.append((gates.to(cuda_device), tokens.to(cuda_device), scan_oracle.scan(gates.numpy(), tokens.numpy())))
    _native.set_option(_native.OPT_TEST_EPOCH_BITS, 2)
    try:
        for i in range(12):
            g, x, want = cases[i % 2]
            out = torch.empty_like(x)
            _native.forward(g, x, out)
            assert rel_err(to_np(out), want) <= 1e-5, i
        _native.check_status(cuda_device)
    finally:
        _native.set_option(_native.OPT_TEST_EPOCH_BITS, 17)
