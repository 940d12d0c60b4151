"""Every sequence length from 1 to 800, for 1, 2 and 5 rows, in fp32, bf16 and complex64,
forward, reversed forward and fused backward, against the CPU oracle; and rows of about one
and two tiles at 300 rows (the kernels that group several rows into one item).  Small shapes
reach every boundary case of the tile arithmetic (rows inside a lane, rows ending inside a
tile, ragged last tiles, unaligned rows with the element-wise loader); an out-of-range access
shows up as a wrong value next to the touched rows, which is what stands in for a memory
checker here."""
import numpy as np
import pytest
import torch

from helpers import complex_inputs, real_inputs, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.complex64: 1e-5, torch.bfloat16: 2.0 ** -8}
GUARD = 64      # elements of padding around every output, checked to be untouched


def _inputs(dtype, shape, seed):
    if dtype == torch.complex64:
        return complex_inputs(seed, shape, law="easy")
    return real_inputs(seed, shape, dtype=dtype)


def _up(t):
    return t.numpy() if t.dtype in (torch.float32, torch.complex64) else t.float().numpy()


def _guarded(like, dev):
    """An output buffer with guard elements on both sides; returns (whole, view)."""
    n = like.numel()
    whole = torch.full((n + 2 * GUARD,), 7.0, dtype=like.dtype, device=dev)
    return whole, whole[GUARD:GUARD + n].view(like.shape)


def _guards_intact(whole):
    w = whole.float() if whole.dtype == torch.bfloat16 else whole
    return bool((w[:GUARD] == 7.0).all()) and bool((w[-GUARD:] == 7.0).all())


def _one_shape(dev, dtype, rows, T, seed):
    from accelerated_scan import _native

    gates, tokens, grad_out = _inputs(dtype, (1, rows, T), seed)
    tol = TOL[dtype]
    g, x, go = gates.to(dev), tokens.to(dev), grad_out.to(dev)
    want = scan_oracle.scan(_up(gates), _up(tokens))
    want_rev = scan_oracle.scan(_up(gates), _up(tokens), reverse=True)
    w_out, out = _guarded(x, dev)
    w_rev, rev = _guarded(x, dev)
    _native.forward(g, x, out)
    _native.forward(g, x, rev, reverse=True)
    states = to_np(out) if dtype == torch.bfloat16 else want
    want_dg, want_dx = scan_oracle.scan_backward(_up(gates), states, _up(grad_out))
    w_dg, dg = _guarded(x, dev)
    w_dx, dx = _guarded(x, dev)
    _native.backward(g, out, go, dg, dx)
    errs = (rel_err(to_np(out), want), rel_err(to_np(rev), want_rev), rel_err(to_np(dx), want_dx),
            rel_err(to_np(dg), want_dg))
    ok = all(e <= tol for e in errs) and all(_guards_intact(w) for w in (w_out, w_rev, w_dg, w_dx))
    return ok, errs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.complex64])
@pytest.mark.parametrize("rows", [1, 2, 5])
def test_every_length_up_to_800(cuda_device, dtype, rows):
    from accelerated_scan import _native

    bad = []
    for T in range(1, 801):
        ok, errs = _one_shape(cuda_device, dtype, rows, T, seed=T)
        if not ok:
            bad.append((T, errs))
    _native.check_status(cuda_device)
    assert not bad, bad[:5]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.complex64])
def test_rows_of_about_one_and_two_tiles_at_300_rows(cuda_device, dtype):
    from accelerated_scan import _native

    code = _native.DTYPE_CODE[dtype]
    tile = _native.plan(300, 100, code, _native.KIND_FORWARD)["tile_elems"]
    bad = []
    for T in (tile - 1, tile, tile + 1, 2 * tile - 1, 2 * tile, 2 * tile + 1):
        ok, errs = _one_shape(cuda_device, dtype, 300, T, seed=T)
        if not ok:
            bad.append((T, errs))
    _native.check_status(cuda_device)
    assert not bad, bad
