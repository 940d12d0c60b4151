"""complex64 CUDA kernels against the CPU oracle.  Mirrors the reference's
tests/tests_eq_complex.py: seeds, input laws (easy / hard radius), real inputs,
three losses, atol 1e-5 / rtol 1e-4."""
import numpy as np
import pytest
import torch

from helpers import complex_inputs, golden_files, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

SEEDS = [1, 11, 22]                                            # tests_eq_complex.py:7
SEQLENS = [2 ** i for i in range(12, 18)] + [16323, 8000, 33753, 127323]   # tests_eq_complex.py:8
ATOL, RTOL = 1e-5, 1e-4                                        # tests_eq_complex.py:23
REL = 1e-5


def loss_real_mean(out):
    return out.real.mean()


def loss_last_sum(out):
    return out[:, :, -1].real.sum() + out[:, :, -1].imag.sum()


def loss_abs_sq_mean(out):
    return out.abs().square().mean()


LOSSES = [loss_real_mean, loss_last_sum, loss_abs_sq_mean]


def _cplx():
    import accelerated_scan.complex as cplx
    return cplx


@pytest.mark.parametrize("path", golden_files("complex_"))
def test_golden_vectors(cuda_device, path):
    cplx = _cplx()
    d = np.load(path)
    forget = torch.from_numpy(d["forget"]).to(cuda_device).requires_grad_(True)
    inputs = torch.from_numpy(d["inputs"]).to(cuda_device).requires_grad_(True)
    out = cplx.scan(forget, inputs)
    np.testing.assert_allclose(to_np(out), d["out"], atol=ATOL, rtol=RTOL)
    assert rel_err(to_np(out), d["out"]) <= REL
    out.backward(torch.from_numpy(d["grad_out"]).to(cuda_device))
    assert inputs.grad.dtype == inputs.dtype
    np.testing.assert_allclose(to_np(forget.grad), d["d_forget"], atol=ATOL, rtol=RTOL)
    np.testing.assert_allclose(to_np(inputs.grad), d["d_inputs"], atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("seed", SEEDS[:1])
@pytest.mark.parametrize("seqlen", SEQLENS)
@pytest.mark.parametrize("law", ["easy", "hard"])
def test_complex_forward_real_inputs(cuda_device, seed, seqlen, law):
    cplx = _cplx()
    forget, inputs, _ = complex_inputs(seed, (1, 16, seqlen), law=law, real_tokens=True)
    want = scan_oracle.scan(forget.numpy(), inputs.numpy())
    out = cplx.scan(forget.to(cuda_device), inputs.to(cuda_device))
    assert out.dtype == torch.complex64
    assert rel_err(to_np(out), want) <= REL
    np.testing.assert_allclose(to_np(out), want, atol=ATOL, rtol=RTOL)


@pytest.mark.parametrize("seed", SEEDS)
@pytest.mark.parametrize("seqlen", [4096, 8000, 16323, 65536])
@pytest.mark.parametrize("law", ["easy", "hard"])
@pytest.mark.parametrize("loss_fn", LOSSES)
def test_complex_backward_losses(cuda_device, seed, seqlen, law, loss_fn):
    """The upstream gradient of each loss is taken from torch autograd on the GPU
    output, then the same gradient drives the oracle's backward."""
    cplx = _cplx()
    forget, inputs, _ = complex_inputs(seed, (1, 8, seqlen), law=law, real_tokens=True)
    f = forget.to(cuda_device).requires_grad_(True)
    x = inputs.to(cuda_device).requires_grad_(True)
    out = cplx.scan(f, x)
    (grad_out,) = torch.autograd.grad(loss_fn(out), out, retain_graph=True)
    out.backward(grad_out)
    want = scan_oracle.scan(forget.numpy(), inputs.numpy())
    want_df, want_dx = scan_oracle.scan_backward(forget.numpy(), want, to_np(grad_out))
    assert x.grad.dtype == torch.float32
    scale_f = max(float(np.abs(want_df).max()), 1e-30)
    scale_x = max(float(np.abs(want_dx.real).max()), 1e-30)
    assert float(np.abs(to_np(f.grad) - want_df).max()) / scale_f <= 2e-5
    assert float(np.abs(to_np(x.grad) - want_dx.real).max()) / scale_x <= 2e-5


@pytest.mark.parametrize("seqlen", [1, 2, 3, 63, 64, 65, 191, 192, 193, 1000, 1001])
@pytest.mark.parametrize("rows", [(1, 1), (2, 5)])
def test_complex_small_and_ragged(cuda_device, seqlen, rows):
    cplx = _cplx()
    forget, inputs, grad_out = complex_inputs(3, (rows[0], rows[1], seqlen), law="cfg4")
    want = scan_oracle.scan(forget.numpy(), inputs.numpy())
    want_df, want_dx = scan_oracle.scan_backward(forget.numpy(), want, grad_out.numpy())
    f = forget.to(cuda_device).requires_grad_(True)
    x = inputs.to(cuda_device).requires_grad_(True)
    out = cplx.scan(f, x)
    out.backward(grad_out.to(cuda_device))
    assert rel_err(to_np(out), want) <= REL
    assert rel_err(to_np(x.grad), want_dx) <= REL
    assert rel_err(to_np(f.grad), want_df) <= REL


def test_reference_config_4(cuda_device):
    """complex64 forward+backward, gates r*exp(i*theta), r ~ U(0.9, 0.999), theta ~ U(-pi, pi),
    complex normal tokens and grad_out; (4, 1024, 16384) cut to (4, 64, 16384) for the CPU oracle."""
    cplx = _cplx()
    forget, inputs, grad_out = complex_inputs(0, (4, 64, 16384), law="cfg4")
    want = scan_oracle.scan(forget.numpy(), inputs.numpy())
    want_df, want_dx = scan_oracle.scan_backward(forget.numpy(), want, grad_out.numpy())
    f = forget.to(cuda_device).requires_grad_(True)
    x = inputs.to(cuda_device).requires_grad_(True)
    out = cplx.scan(f, x)
    out.backward(grad_out.to(cuda_device))
    np.testing.assert_allclose(to_np(out), want, atol=ATOL, rtol=RTOL)
    assert rel_err(to_np(out), want) <= REL
    assert rel_err(to_np(x.grad), want_dx) <= REL
    assert rel_err(to_np(f.grad), want_df) <= REL


def test_forget_must_be_complex(cuda_device):
    cplx = _cplx()
    g = torch.rand(1, 2, 32, device=cuda_device)
    with pytest.raises(TypeError):
        cplx.scan(g, g.clone())


def test_triton_style_launchers(cuda_device):
    """forward_scan[(B, C)](...) / backward_scan[(B, C)](...) keep the call form the
    reference's benchmark uses (tests/bench_complex.py:31-45)."""
    cplx = _cplx()
    B, C, T = 1, 4, 2048
    forget, inputs, grad_out = complex_inputs(2, (B, C, T), law="cfg4")
    want = scan_oracle.scan(forget.numpy(), inputs.numpy())
    f, x, go = forget.to(cuda_device), inputs.to(cuda_device), grad_out.to(cuda_device)
    states = torch.empty_like(x)
    cplx.forward_scan[(B, C)](torch.view_as_real(f), torch.view_as_real(x), torch.view_as_real(states), seqlen=T)
    assert rel_err(to_np(states), want) <= REL
    d_f, d_x = torch.empty_like(f), torch.empty_like(x)
    cplx.backward_scan[(B, C)](torch.view_as_real(f), torch.view_as_real(states), torch.view_as_real(go),
                               torch.view_as_real(d_x), torch.view_as_real(d_f), seqlen=T)
    want_df, want_dx = scan_oracle.scan_backward(forget.numpy(), want, grad_out.numpy())
    assert rel_err(to_np(d_x), want_dx) <= REL
    assert rel_err(to_np(d_f), want_df) <= REL


@pytest.mark.parametrize("rows,seqlen,fused", [(2000, 4096, True), (8, 40000, True), (300, 20000, True),
                                               (4, 16323, False), (6, 1002, False)])
def test_real_tokens_fused_into_the_kernel(cuda_device, rows, seqlen, fused):
    """Real inputs go into the complex kernel as fp32 (no complex copy) whenever the rows are
    16-byte aligned in both streams (seqlen % 4 == 0); other shapes report "unsupported" and
    complex.scan promotes the tokens as the reference does.  Both give the same answer."""
    from accelerated_scan import _native

    cplx = _cplx()
    forget, inputs, _ = complex_inputs(21, (1, rows, seqlen), law="cfg4", real_tokens=True)
    want = scan_oracle.scan(forget.numpy(), inputs.numpy())
    f, x = forget.to(cuda_device), inputs.to(cuda_device)
    out = torch.empty_like(f)
    assert _native.forward_complex_real_tokens(f, x, out) == fused
    if fused:
        assert rel_err(to_np(out), want) <= REL
        rev = torch.empty_like(f)
        assert _native.forward_complex_real_tokens(f, x, rev, reverse=True)
        assert rel_err(to_np(rev), scan_oracle.scan(forget.numpy(), inputs.numpy(), reverse=True)) <= REL
    assert rel_err(to_np(cplx.scan(f, x)), want) <= REL
    # backward: only the real part of the token gradient is written, as fp32
    g = torch.Generator().manual_seed(22)
    grad_out = torch.complex(torch.randn(1, rows, seqlen, generator=g), torch.randn(1, rows, seqlen, generator=g))
    want_df, want_dx = scan_oracle.scan_backward(forget.numpy(), want, grad_out.numpy())
    states = torch.from_numpy(want).to(cuda_device)
    d_f = torch.empty_like(f)
    d_x = torch.full((1, rows, seqlen), float("nan"), dtype=torch.float32, device=cuda_device)
    assert _native.backward_complex_real_tokens(f, states, grad_out.to(cuda_device), d_f, d_x) == fused
    if fused:
        assert rel_err(to_np(d_f), want_df) <= REL
        assert rel_err(to_np(d_x), want_dx.real) <= REL
