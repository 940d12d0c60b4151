"""Every launch plan of the planner against the CPU oracle: the stream kernel with
chained segments, the look-back plan (fewer rows than SMs) and the team plan (fewer rows
than warps, 2..12 warps per item), for all kinds, dtypes and the seeded forms.  The plan
a shape gets is asserted, so a planner change cannot silently drop the coverage."""
import numpy as np
import pytest
import torch

from helpers import complex_inputs, real_inputs, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.complex64: 1e-5, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -10}


def _inputs(dtype, shape, seed=13):
    if dtype == torch.complex64:
        return complex_inputs(seed, shape, law="cfg4")
    law = "uniform" if dtype == torch.float16 else "near_one"
    return real_inputs(seed, shape, law=law, dtype=dtype)


def _up(t):
    return t.numpy() if t.dtype in (torch.float32, torch.complex64) else t.float().numpy()


# rows, seqlen, expected plan kernel (0 stream, 1 look-back, 2 team), expected team size of the
# backward (12 warps per CTA) and of the forward (16 warps per CTA)
CASES = [
    (7200, 13000, 0, 1, 1),      # more than four rows per warp: chained stream kernel
    (4000, 16384, 2, 2, 2),      # two to four rows per warp, rows long enough to split: teams of two
    (2000, 8192, 2, 2, 2),       # about one row per warp: teams of two
    (1024, 16384, 2, 2, 4),      # config-5-like
    (700, 9000, 2, 3, 4),
    (450, 12288, 2, 4, 8),
    (300, 20000, 2, 6, 8),
    (160, 33000, 2, 12, 16),
    (100, 50000, 1, 1, 1),       # clearly fewer rows than SMs: look-back
    (3, 400000, 1, 1, 1),
]


@pytest.mark.parametrize("rows,seqlen,kernel,team,team_fwd", CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.complex64])
def test_plan_parity(cuda_device, rows, seqlen, kernel, team, team_fwd, dtype):
    from accelerated_scan import _native

    if dtype == torch.complex64:
        seqlen = seqlen // 2          # same bytes per row
    code = _native.DTYPE_CODE[dtype]
    for kind in (_native.KIND_FORWARD, _native.KIND_BACKWARD):
        pl = _native.plan(rows, seqlen, code, kind)
        # the forward takes the look-back plan up to 3/2 rows per SM, the backward up to 3/4
        want_kernel = 1 if (kernel == 2 and kind == _native.KIND_FORWARD and rows < 222) else kernel
        assert pl["kernel"] == want_kernel, pl
        if want_kernel == 2:
            assert pl["team_size"] == (team_fwd if kind == _native.KIND_FORWARD else team), pl
            assert pl["warps_per_cta"] == (16 if kind == _native.KIND_FORWARD else 12), pl
        else:
            assert pl["team_size"] == 1, pl
    shape = (1, rows, seqlen)
    gates, tokens, grad_out = _inputs(dtype, shape)
    want = scan_oracle.scan(_up(gates), _up(tokens))
    want_rev = scan_oracle.scan(_up(gates), _up(tokens), reverse=True)
    g, x, go = gates.to(cuda_device), tokens.to(cuda_device), grad_out.to(cuda_device)
    out, rev = torch.empty_like(x), torch.empty_like(x)
    _native.forward(g, x, out)
    _native.forward(g, x, rev, reverse=True)
    tol = TOL[dtype]
    assert rel_err(to_np(out), want) <= tol
    assert rel_err(to_np(rev), want_rev) <= tol
    states = to_np(out) if dtype == torch.bfloat16 else want
    want_dg, want_dx = scan_oracle.scan_backward(_up(gates), states, _up(grad_out))
    dg, dx = torch.empty_like(x), torch.empty_like(x)
    _native.backward(g, out, go, dg, dx)
    assert rel_err(to_np(dx), want_dx) <= tol
    assert rel_err(to_np(dg), want_dg) <= tol
    _native.check_status(cuda_device)


@pytest.mark.parametrize("rows,seqlen", [(1024, 12000), (300, 20000), (100, 30000), (2000, 6000), (7200, 6000)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64])
def test_plan_seeded_forms(cuda_device, rows, seqlen, dtype):
    """carry_in, halo_gate_right and halo_state_left under every plan: scanning the second
    half of a sequence seeded with the first half's state equals the unsharded result."""
    from accelerated_scan import _native, sharded

    shape = (1, rows, 2 * seqlen)
    gates, tokens, grad_out = _inputs(dtype, shape, seed=29)
    want = scan_oracle.scan(_up(gates), _up(tokens))
    want_dg, want_dx = scan_oracle.scan_backward(_up(gates), want, _up(grad_out))
    cdt = sharded.compute_dtype(dtype)
    half = lambda t, h: t[..., h * seqlen:(h + 1) * seqlen].contiguous().to(cuda_device)
    g0, g1, x0, x1, go0, go1 = half(gates, 0), half(gates, 1), half(tokens, 0), half(tokens, 1), half(grad_out, 0), half(grad_out, 1)
    s0 = torch.empty_like(x0)
    _native.forward(g0, x0, s0)
    carry = s0[0, :, -1].to(cdt).contiguous()
    s1 = torch.empty_like(x1)
    _native.forward(g1, x1, s1, carry_in=carry)
    got = torch.cat([s0, s1], dim=-1)
    assert rel_err(to_np(got), want) <= 1e-5
    # backward of the second half needs the state before it; the first half needs the adjoint after it
    dg1, dx1 = torch.empty_like(x1), torch.empty_like(x1)
    _native.backward(g1, s1, go1, dg1, dx1, halo_state_left=carry)
    g_in = dx1[0, :, 0].to(cdt).contiguous()
    first_gate = g1[0, :, 0].to(cdt).contiguous()
    dg0, dx0 = torch.empty_like(x0), torch.empty_like(x0)
    _native.backward(g0, s0, go0, dg0, dx0, carry_in=g_in, halo_gate_right=first_gate)
    assert rel_err(to_np(torch.cat([dx0, dx1], dim=-1)), want_dx) <= 1e-5
    assert rel_err(to_np(torch.cat([dg0, dg1], dim=-1)), want_dg) <= 1e-5
    _native.check_status(cuda_device)


def test_small_workspace_steps_down_to_chained(cuda_device):
    """A caller-supplied workspace that only fits the chained plan (256 + 32*rows bytes)
    still gives the right answer for a shape whose preferred plan is look-back."""
    import ctypes
    from accelerated_scan import _native

    rows, T = 16, 120000
    gates, tokens, _ = real_inputs(31, (1, rows, T), grad=False)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    g, x = gates.to(cuda_device), tokens.to(cuda_device)
    out = torch.empty_like(x)
    ws = torch.zeros(256 + 32 * rows, dtype=torch.uint8, device=cuda_device)
    assert _native.lib.ascan_workspace_bytes(rows, T, _native.F32, 0) > ws.numel()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = _native.lib.ascan_forward(p(g), p(x), p(out), rows, T, _native.F32, 0, None, p(ws), ws.numel(),
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    assert rel_err(to_np(out), want) <= 1e-5
    out2 = torch.empty_like(x)
    rc = _native.lib.ascan_forward(p(g), p(x), p(out2), rows, T, _native.F32, 0, None, None, 0,
                                   ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    assert rel_err(to_np(out2), want) <= 1e-5


@pytest.mark.parametrize("lb_tiles", [1, 3, 4])
def test_lookback_with_other_segment_lengths(cuda_device, lb_tiles):
    """The look-back plan with other segment lengths than the default (1, 3 and 4 tiles per segment): same results, forward and backward."""
    from accelerated_scan import _native

    default_tiles = _native.get_option(_native.OPT_LOOKBACK_TILES)
    _native.set_option(_native.OPT_LOOKBACK_TILES, lb_tiles)
    try:
        _lookback_case(cuda_device)
    finally:
        _native.set_option(_native.OPT_LOOKBACK_TILES, default_tiles)


def _lookback_case(cuda_device):
    from accelerated_scan import _native

    rows, T = 5, 100000
    assert _native.plan(rows, T, _native.F32, _native.KIND_FORWARD)["kernel"] == 1
    gates, tokens, grad_out = real_inputs(33, (1, rows, T), law="near_one")
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad_out.numpy())
    g, x, go = (t.to(cuda_device) for t in (gates, tokens, grad_out))
    out = torch.empty_like(x)
    _native.forward(g, x, out)
    assert rel_err(to_np(out), want) <= 1e-5
    dg, dx = torch.empty_like(x), torch.empty_like(x)
    _native.backward(g, out, go, dg, dx)
    assert rel_err(to_np(dx), want_dx) <= 1e-5
    assert rel_err(to_np(dg), want_dg) <= 1e-5
    _native.check_status(cuda_device)


# Lengths around the boundaries of the look-back plan's decomposition (fp32: tiles of 384 steps,
# parts of 2 tiles, segments of up to 15 parts forward and 11 backward): rows shorter than a
# full team, exactly one segment, one step or one tile more, workers whose part is empty in
# the last segment, a ragged last tile.  (Multiples of four steps: rows of whole 16-byte chunks.)
LOOKBACK_LENGTHS = [1156, 1536, 1540, 2308, 4608, 8444, 8448, 8452, 11516, 11520, 11524, 11908, 16900, 23040, 23044, 34568]


@pytest.mark.parametrize("rows", [1, 3])
@pytest.mark.parametrize("T", LOOKBACK_LENGTHS)
def test_lookback_segment_boundaries(cuda_device, rows, T):
    """Forward, reversed forward, seeded forward and fused backward of the look-back plan against the CPU oracle."""
    from accelerated_scan import _native

    for kind in (_native.KIND_FORWARD, _native.KIND_BACKWARD):
        pl = _native.plan(rows, T, _native.F32, kind)
        assert pl["kernel"] == 1, pl
        assert (pl["segs_per_row"] - 1) * pl["seg_elems"] < T <= pl["segs_per_row"] * pl["seg_elems"]
    gates, tokens, grad_out = real_inputs(1000 + T, (1, rows, T), law="near_one")
    seed = torch.linspace(-1.0, 1.0, rows)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_rev = scan_oracle.scan(gates.numpy(), tokens.numpy(), reverse=True)
    # a scan started from a state is the plain scan plus the running product of the gates times that state
    want_seeded = want + np.cumprod(gates.numpy().astype(np.float64), axis=-1) * seed.numpy().astype(np.float64).reshape(1, rows, 1)
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad_out.numpy())
    g, x, go = (t.to(cuda_device) for t in (gates, tokens, grad_out))
    out = torch.empty_like(x)
    _native.forward(g, x, out)
    assert rel_err(to_np(out), want) <= 1e-5
    dg, dx = torch.empty_like(x), torch.empty_like(x)
    _native.backward(g, out, go, dg, dx)
    assert rel_err(to_np(dx), want_dx) <= 1e-5
    assert rel_err(to_np(dg), want_dg) <= 1e-5
    _native.forward(g, x, out, reverse=True)
    assert rel_err(to_np(out), want_rev) <= 1e-5
    _native.forward(g, x, out, carry_in=seed.to(cuda_device))
    assert rel_err(to_np(out), want_seeded) <= 1e-5
    _native.check_status(cuda_device)
