"""ascan_forward_no_alloc: the forward scan for callers that cannot provide scratch
memory (hosts that reserved all device memory up front, loops that must not call
cudaMalloc, bindings that only own their input and output buffers).  Its scratch is a
fixed array inside the library, shared by every call on the device.

The test calls the entry point through the C ABI twice in a row and compares each
result with the regular entry point (caller-supplied workspace) on the same inputs and
with the CPU oracle; the second call runs on the leftovers of the first.  Collected last
on purpose."""
import ctypes

import pytest
import torch

from helpers import real_inputs, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

FP32_REL = 1e-5
BF16_REL = 2.0 ** -8       # against the oracle run in fp32 on the bf16-rounded inputs


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


@pytest.mark.parametrize("shape,dtype", [((2, 32, 65536), torch.float32), ((1, 48, 160000), torch.bfloat16),
                                         ((1, 8, 65536), torch.float32)])
def test_no_alloc_matches_workspace_entry_point(cuda_device, shape, dtype):
    from accelerated_scan import _native

    lib = _native.lib
    rows, T = shape[0] * shape[1], shape[2]
    code = _native.DTYPE_CODE[dtype]
    # long rows: both entry points split them into segments and pass carries through scratch
    assert _native.plan(rows, T, code, _native.KIND_FORWARD, lookback=False)["segs_per_row"] > 1
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    for call, seed in enumerate((21, 22)):
        gates, tokens, _ = real_inputs(seed, shape, law="near_one", dtype=dtype, grad=False)
        g, x = gates.to(cuda_device), tokens.to(cuda_device)
        up = (lambda t: t.numpy()) if dtype == torch.float32 else (lambda t: t.float().numpy())
        for reverse in (0, 1):
            oracle = scan_oracle.scan(up(gates), up(tokens), reverse=bool(reverse))
            want = torch.empty_like(x)
            _native.forward(g, x, want, reverse=bool(reverse))
            got = torch.full_like(x, float("nan"))
            rc = lib.ascan_forward_no_alloc(_ptr(g), _ptr(x), _ptr(got), rows, T, code, reverse, stream)
            assert rc == 0, _native.strerror(rc)
            torch.cuda.synchronize(cuda_device)
            tol = FP32_REL if dtype == torch.float32 else BF16_REL
            assert rel_err(to_np(got), oracle) <= tol, (call, reverse)
            # (the two entry points may plan differently -- the built-in scratch can be too small
            # for a plan's records -- so they agree to rounding, not bit for bit: for 16-bit
            # storage at most one unit in the last place of the stored value)
            pair_tol = FP32_REL if dtype == torch.float32 else 2.0 ** -7
            assert rel_err(to_np(got), to_np(want)) <= pair_tol, (call, reverse)


def test_no_alloc_rejects_too_many_rows(cuda_device):
    from accelerated_scan import _native

    x = torch.zeros(8, device=cuda_device)
    rc = _native.lib.ascan_forward_no_alloc(_ptr(x), _ptr(x), _ptr(x), 16385, 8, _native.F32, 0, None)
    assert rc == 7
    assert "16384" in _native.strerror(rc)
    assert _native.lib.ascan_forward_no_alloc(_ptr(x), _ptr(x), _ptr(x), 4, 0, _native.F32, 0, None) == 1
