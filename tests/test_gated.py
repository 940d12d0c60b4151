"""Scan with sigmoid gates fused into the kernels against the CPU oracle fed with
sigmoid(gate_logits): forward, gradient of the logits, gradient of the tokens."""
import numpy as np
import pytest
import torch

from helpers import rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

TOL = {torch.float32: 1e-5, torch.bfloat16: 2.0 ** -7, torch.float16: 2.0 ** -10}


def _inputs(seed, shape, dtype, law):
    g = torch.Generator().manual_seed(seed)
    if law == "normal":          # gates spread over (0, 1)
        logits = 2.0 * torch.randn(*shape, generator=g)
    else:                        # gates in (0.998, 0.9998): long memory
        logits = 6.0 + 3.0 * torch.rand(*shape, generator=g)
    tokens = torch.rand(*shape, generator=g)
    grad_out = torch.randn(*shape, generator=g)
    return logits.to(dtype), tokens.to(dtype), grad_out.to(dtype)


def _oracle(logits, tokens, grad_out):
    z = logits.double().numpy()
    s = (1.0 / (1.0 + np.exp(-z))).astype(np.float32)
    x = tokens.float().numpy()
    out = scan_oracle.scan(s, x)
    d_gates, d_tokens = scan_oracle.scan_backward(s, out, grad_out.float().numpy())
    d_logits = d_gates * (s * (1.0 - s))
    return out, d_logits, d_tokens, d_gates


def _logit_grad_err(got, want, d_gates):
    """d_logits = d_gates * s * (1 - s) is formed from the fp32 gate s, as torch's own
    sigmoid backward does.  For gates close to one, one ulp of s moves 1 - s by 2^-24 / (1 - s)
    of its value, so the comparison allows the gate to differ from the oracle's by 4 ulp
    (the kernel's sigmoid uses the approximate exp2 and reciprocal instructions) on top of
    the usual max-norm tolerance."""
    slack = 4.0 * 2.0 ** -23 * np.abs(d_gates.astype(np.float64))
    excess = np.maximum(np.abs(got.astype(np.float64) - want.astype(np.float64)) - slack, 0.0)
    return float(excess.max() / max(np.abs(want).max(), 1e-30))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("shape,fused", [
    ((2, 3, 4096), True),         # whole rows, static dealing
    ((1, 5, 3001 * 8), True),     # ragged last tile
    ((2, 700, 2048), True),       # more rows than warps on a B200: tickets
    ((1, 4, 40000), True),        # rows split into chained segments
    ((2, 3, 100), None),          # short rows are grouped: no fused kernel, falls back
    ((1, 3, 1001), None),         # rows not 16-byte aligned: falls back
])
@pytest.mark.parametrize("law", ["normal", "long_memory"])
def test_sigmoid_gate_scan_matches_oracle(cuda_device, dtype, shape, fused, law):
    from accelerated_scan import _native, gated

    if dtype == torch.float16 and law == "long_memory" and shape[-1] > 1024:
        pytest.skip("states overflow fp16")
    logits, tokens, grad_out = _inputs(5, shape, dtype, law)
    want_out, want_dz, want_dx, want_da = _oracle(logits, tokens, grad_out)
    z = logits.to(cuda_device).requires_grad_(True)
    x = tokens.to(cuda_device).requires_grad_(True)
    if fused:
        probe = torch.empty_like(x)
        assert _native.forward_sigmoid_gates(z.detach(), x.detach(), probe), "expected the fused kernel for this shape"
    out = gated.scan(z, x)
    out.backward(grad_out.to(cuda_device))
    tol = TOL[dtype]
    assert rel_err(to_np(out), want_out) <= tol
    assert rel_err(to_np(x.grad), want_dx) <= tol
    assert _logit_grad_err(to_np(z.grad), want_dz, want_da) <= tol
    _native.check_status(cuda_device)


def test_fused_and_unfused_agree_fp32(cuda_device):
    from accelerated_scan import gated, warp

    logits, tokens, grad_out = _inputs(6, (2, 300, 8192), torch.float32, "normal")
    z1 = logits.to(cuda_device).requires_grad_(True)
    x1 = tokens.to(cuda_device).requires_grad_(True)
    z2 = logits.to(cuda_device).requires_grad_(True)
    x2 = tokens.to(cuda_device).requires_grad_(True)
    g = grad_out.to(cuda_device)
    out1 = gated.scan(z1, x1)
    out1.backward(g)
    out2 = warp.scan(torch.sigmoid(z2), x2)
    out2.backward(g)
    assert rel_err(to_np(out1), to_np(out2)) <= 2e-6
    assert rel_err(to_np(x1.grad), to_np(x2.grad)) <= 2e-6
    assert rel_err(to_np(z1.grad), to_np(z2.grad)) <= 2e-6


def test_rejects_complex(cuda_device):
    from accelerated_scan import gated

    z = torch.zeros(1, 1, 64, dtype=torch.complex64, device=cuda_device)
    with pytest.raises(RuntimeError):
        gated.scan(z, z)
