"""Bounded device-side waits: a wait that can never be satisfied runs out, the kernel still
finishes, the status word reports it, and the context stays usable.  The failure is made by
a test hook that drops ONE carry hand-over (nothing faults, traps or hangs)."""
import os

import pytest
import torch

from helpers import real_inputs, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_context_survives(cuda_device):
    from accelerated_scan import _native

    rows, T = 7200, 16000          # chained stream plan: more than four rows per warp, several segments per row
    pl = _native.plan(rows, T, _native.F32, _native.KIND_FORWARD)
    assert pl["kernel"] == 0 and pl["segs_per_row"] > 1 and pl["dynamic"] == 1
    gates, tokens, _ = real_inputs(2, (1, rows, T), grad=False)
    g, x = gates.to(cuda_device), tokens.to(cuda_device)
    out = torch.empty_like(x)
    _native.check_status(cuda_device)                     # clean before
    os.environ["ASCAN_TEST_DROP_CARRY"] = "1"
    try:
        _native.forward(g, x, out)                        # row 0 loses the state between two segments
        with pytest.raises(RuntimeError, match="bounded device-side wait"):
            _native.check_status(cuda_device)
    finally:
        del os.environ["ASCAN_TEST_DROP_CARRY"]
    # the status word was cleared by the check, the workspace rearmed itself: a normal call is right
    _native.forward(g, x, out)
    _native.check_status(cuda_device)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    assert rel_err(to_np(out), want) <= 1e-5
