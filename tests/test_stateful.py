"""scan with an initial state: chunked scanning equals scanning the whole sequence, and the
gradients (including the one of the initial state) match torch autograd through a plain
loop of the recurrence."""
import numpy as np
import pytest
import torch

from helpers import complex_inputs, real_inputs, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu


def _loop_scan(gates, tokens, x0):
    xs = []
    x = x0
    for t in range(gates.shape[-1]):
        x = gates[..., t] * x + tokens[..., t]
        xs.append(x)
    return torch.stack(xs, dim=-1)


@pytest.mark.parametrize("cplx", [False, True])
def test_gradients_match_autograd_loop(cuda_device, cplx):
    from accelerated_scan import stateful

    shape = (2, 3, 200)
    if cplx:
        gates, tokens, grad_out = complex_inputs(4, shape, law="cfg4")
        x0 = torch.complex(torch.randn(2, 3), torch.randn(2, 3))
    else:
        gates, tokens, grad_out = real_inputs(4, shape)
        x0 = torch.randn(2, 3)
    ref_in = [t.clone().double().requires_grad_(True) if not cplx else t.clone().to(torch.complex128).requires_grad_(True)
              for t in (gates, tokens, x0)]
    ref = _loop_scan(*ref_in)
    ref.backward(grad_out.to(ref.dtype))
    dev_in = [t.to(cuda_device).requires_grad_(True) for t in (gates, tokens, x0)]
    out = stateful.scan(*dev_in)
    out.backward(grad_out.to(cuda_device))
    assert rel_err(to_np(out), ref.detach().numpy()) <= 1e-5
    for got, want in zip(dev_in, ref_in):
        assert rel_err(to_np(got.grad), want.grad.numpy()) <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("seqlen,chunk", [(4096, 1000), (70000, 16384)])
def test_chunked_equals_whole(cuda_device, dtype, seqlen, chunk):
    from accelerated_scan import stateful

    gates, tokens, _ = real_inputs(8, (1, 6, seqlen), law="near_one", dtype=dtype, grad=False)
    want = scan_oracle.scan(gates.float().numpy(), tokens.float().numpy())
    g, x = gates.to(cuda_device), tokens.to(cuda_device)
    state = None
    parts = []
    for lo in range(0, seqlen, chunk):
        out = stateful.scan(g[..., lo:lo + chunk].contiguous(), x[..., lo:lo + chunk].contiguous(), state)
        state = out[..., -1].float()
        parts.append(out)
    got = torch.cat(parts, dim=-1)
    # bf16: every chunk boundary rounds the carried state once more
    # bf16: the state handed on is out[..., -1], already rounded to bf16; with gates near one
    # each of the four chunk boundaries adds up to 2^-9 of relative error that decays slowly
    tol = 1e-5 if dtype == torch.float32 else 2.0 ** -6
    assert rel_err(to_np(got), want) <= tol


def test_none_state_is_the_drop_in_scan(cuda_device):
    from accelerated_scan import stateful, warp

    gates, tokens, _ = real_inputs(1, (1, 4, 512), grad=False)
    g, x = gates.to(cuda_device), tokens.to(cuda_device)
    assert torch.equal(stateful.scan(g, x), warp.scan(g, x))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.complex64])
@pytest.mark.parametrize("shape", [(2, 3, 1), (1, 5, 777), (2, 160, 3000), (1, 2, 300000)])
@pytest.mark.parametrize("with_state", [False, True])
def test_final_state_is_the_last_column_of_the_scan(cuda_device, dtype, shape, with_state):
    from accelerated_scan import stateful

    if dtype == torch.complex64:
        gates, tokens, _ = complex_inputs(9, shape, law="cfg4")
        x0 = torch.complex(torch.randn(shape[:2]), torch.randn(shape[:2])) if with_state else None
    else:
        gates, tokens, _ = real_inputs(9, shape, law="near_one" if shape[-1] > 2000 else "uniform", dtype=dtype, grad=False)
        x0 = torch.randn(shape[:2]) if with_state else None
    g, x = gates.to(cuda_device), tokens.to(cuda_device)
    s0 = x0.to(cuda_device) if with_state else None
    # the scan writes its states in the storage dtype; the carry-only kernel keeps fp32
    want = stateful.scan(g, x, s0)[..., -1]
    got = stateful.final_state(g, x, s0)
    assert got.shape == shape[:2]
    assert got.dtype == (torch.complex64 if dtype == torch.complex64 else torch.float32)
    tol = 2.0 ** -8 if dtype == torch.bfloat16 else 1e-5
    assert rel_err(to_np(got), to_np(want.to(got.dtype))) <= tol
