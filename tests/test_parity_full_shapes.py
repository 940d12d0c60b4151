"""Parity at the shapes the benchmark numbers are quoted on.  The tensors are too large for
the CPU oracle as a whole, so they are drawn on the GPU and a fixed subset of rows (the first
and last 8 of each batch) is copied back and recomputed by the oracle on the same values.
Mirrors what the reference compares in tests/test_eq.py:26-62 and tests/tests_eq_complex.py:55-86."""
import math

import numpy as np
import pytest
import torch

from helpers import rel_err
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

BAR = {torch.float32: 1e-5, torch.complex64: 1e-5, torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -10}


def _subset(batch, dim, k=8):
    idx = []
    for b in range(batch):
        idx += list(range(b * dim, b * dim + k)) + list(range((b + 1) * dim - k, (b + 1) * dim))
    return idx


def _draw(dev, shape, dtype, law, seed):
    gen = torch.Generator(device=dev).manual_seed(seed)
    if dtype == torch.complex64:
        r = 0.9 + 0.099 * torch.rand(*shape, device=dev, generator=gen)
        th = (2 * torch.rand(*shape, device=dev, generator=gen) - 1) * math.pi
        g = torch.polar(r, th)
        del r, th
        x = torch.complex(torch.randn(*shape, device=dev, generator=gen), torch.randn(*shape, device=dev, generator=gen))
        go = torch.complex(torch.randn(*shape, device=dev, generator=gen), torch.randn(*shape, device=dev, generator=gen))
        return g, x, go
    g = torch.rand(*shape, device=dev, generator=gen)
    if law == "near_one":
        g = 0.999 + 0.001 * g
    x = torch.rand(*shape, device=dev, generator=gen)
    go = torch.randn(*shape, device=dev, generator=gen)
    return g.to(dtype), x.to(dtype), go.to(dtype)


def _check(dev, shape, dtype, law, seed, api):
    from accelerated_scan import _native

    B, C, T = shape
    g, x, go = _draw(dev, shape, dtype, law, seed)
    if api == "autograd":
        import accelerated_scan.complex as cplx
        import accelerated_scan.warp as warp

        gg, xx = g.requires_grad_(True), x.requires_grad_(True)
        out = (cplx.scan if dtype == torch.complex64 else warp.scan)(gg, xx)
        out.backward(go)
        out, dg, dx = out.detach(), gg.grad, xx.grad
        g, x = g.detach(), x.detach()
    else:
        out, dg, dx = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
        _native.forward(g, x, out)
        _native.backward(g, out, go, dg, dx)
    _native.check_status(dev)
    idx = torch.tensor(_subset(B, C), device=dev)
    exact = dtype in (torch.float32, torch.complex64)
    take = lambda t: (t if exact else t.float()).reshape(-1, T).index_select(0, idx).cpu().numpy()[None]
    G, X, GO, O, DG, DX = (take(t) for t in (g, x, go, out, dg, dx))
    want = scan_oracle.scan(G, X)
    want_dg, want_dx = scan_oracle.scan_backward(G, want if exact else O, GO)
    bar = BAR[dtype]
    assert rel_err(O, want) <= bar
    assert rel_err(DX, want_dx) <= bar
    assert rel_err(DG, want_dg) <= bar
    if dtype == torch.complex64:
        # the reference's own tolerance for the complex path (tests/tests_eq_complex.py:23)
        np.testing.assert_allclose(O, want, atol=1e-5 * max(1.0, float(np.abs(want).max())), rtol=1e-4)


def test_headline_shape_bf16(cuda_device):
    """(8, 1536, 65536) bf16: the shape and dtype of the benchmark's headline value."""
    _check(cuda_device, (8, 1536, 65536), torch.bfloat16, "near_one", 101, "native")
    torch.cuda.empty_cache()


def test_headline_shape_fp32(cuda_device):
    _check(cuda_device, (8, 1536, 65536), torch.float32, "near_one", 102, "native")
    torch.cuda.empty_cache()


def test_config2_fp32_through_autograd(cuda_device):
    """(8, 1536, 4096) fp32, gates and tokens U(0,1), grad_out N(0,1)."""
    _check(cuda_device, (8, 1536, 4096), torch.float32, "uniform", 103, "autograd")


def test_config4_complex64_full_shape(cuda_device):
    """(4, 1024, 16384) complex64, gates r*exp(i*theta), r ~ U(0.9, 0.999)."""
    _check(cuda_device, (4, 1024, 16384), torch.complex64, "cfg4", 104, "autograd")
    torch.cuda.empty_cache()


@pytest.mark.parametrize("L", [128, 256, 512, 1024, 2048, 4096, 8192])
def test_length_sweep_shapes_bf16(cuda_device, L):
    """(8, 1536, L) bf16: at 12288 rows the short rows take the kernels that group rows per item."""
    from accelerated_scan import _native

    if L <= 256:
        assert _native.plan(8 * 1536, L, _native.BF16, _native.KIND_FORWARD)["rows_per_item"] > 1
    _check(cuda_device, (8, 1536, L), torch.bfloat16, "near_one", 200 + L, "native")


def test_rows_of_one_four_chunk_tile_fp16(cuda_device):
    """(8, 1536, 1024) fp16: the forward takes four chunks per lane (one 1024-element tile per row)."""
    from accelerated_scan import _native

    assert _native.plan(8 * 1536, 1024, _native.F16, _native.KIND_FORWARD)["chunks_per_lane"] == 4
    assert _native.plan(8 * 1536, 1024, _native.BF16, _native.KIND_FORWARD)["chunks_per_lane"] == 4
    _check(cuda_device, (8, 1536, 1024), torch.float16, "uniform", 301, "native")
