"""Scan with an explicit initial state: x[-1] = initial_state instead of zero.

The reference always starts from zero (warp.py:69-72).  Streaming inference and chunked
training need to continue a sequence: scan a chunk, keep `out[..., -1]`, pass it as the
`initial_state` of the next chunk.  The kernels already take a per-row incoming state
(`carry_in` of `ascan_forward`, `halo_state_left` of `ascan_backward`); this module is
the autograd surface for it.  Works for the real dtypes and complex64.

    out = scan(gates, tokens, initial_state)          # (B, C, T)
    next_state = out[..., -1]                          # differentiable: it is a slice of `out`

When only the last state is wanted (prefill of a streaming model), `final_state` runs the
carry-only kernel (`ascan_reduce_forward`): it reads the two inputs and writes two values
per row, a third less traffic than the scan and no (B, C, T) output tensor.
"""
import torch

from . import _native
from .sharded import compute_dtype


class ScanWithState(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, tokens, initial_state):
        B, C, T = gates.shape
        assert tokens.shape == (B, C, T)
        assert initial_state.shape == (B, C)
        assert gates.is_contiguous()
        assert tokens.is_contiguous()
        if gates.dtype != tokens.dtype:
            raise RuntimeError("gates and tokens must have the same dtype")
        x0 = initial_state.to(compute_dtype(gates.dtype)).contiguous()
        states = torch.empty_like(tokens)
        if states.numel():
            _native.forward(gates, tokens, states, carry_in=x0.reshape(-1))
        ctx.save_for_backward(gates, states, x0)
        ctx.state_dtype = initial_state.dtype
        return states

    @staticmethod
    def backward(ctx, grad_output):
        gates, states, x0 = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        d_gates = torch.empty_like(gates)
        d_tokens = torch.empty_like(gates)
        if gates.numel():
            # d_gates[0] = conj(x[-1]) * g[0] needs the state before the first step
            _native.backward(gates, states, grad_output, d_gates, d_tokens, halo_state_left=x0.reshape(-1))
        # x[0] = gates[0] * x[-1] + tokens[0]  =>  dL/dx[-1] = conj(gates[0]) * g[0]
        d_state = (gates[..., 0].conj() * d_tokens[..., 0]).to(ctx.state_dtype)
        return d_gates, d_tokens, d_state


def scan(gates, tokens, initial_state=None):
    """x[t] = gates[t] * x[t-1] + tokens[t] with x[-1] = initial_state (zeros if None).

    Arguments:
        gates, tokens (torch.Tensor): (B, C, T), CUDA, contiguous, same dtype
            (float32, bfloat16, float16 or complex64).
        initial_state (torch.Tensor, optional): (B, C); any real dtype for real scans,
            complex64 for complex ones.

    Returns:
        (torch.Tensor): (B, C, T); `out[..., -1]` is the state to hand to the next chunk.
    """
    if initial_state is None:
        if gates.dtype == torch.complex64:
            from . import complex as _complex
            return _complex.scan(gates, tokens)
        from . import warp as _warp
        return _warp.scan(gates, tokens)
    return ScanWithState.apply(gates, tokens, initial_state)


def final_state(gates, tokens, initial_state=None):
    """x[T-1] of the scan without materialising x: (B, C) in the accumulation dtype
    (float32 for the real dtypes, complex64 for complex64).  Not differentiable (the
    states that the gradient of the gates needs are never written); use `scan` to train.

    The kernel returns, per row, the product P of the gates and the last state S from a
    zero start; the state from `initial_state` is P * initial_state + S.
    """
    B, C, T = gates.shape
    assert tokens.shape == (B, C, T)
    assert gates.is_contiguous()
    assert tokens.is_contiguous()
    if gates.dtype != tokens.dtype:
        raise RuntimeError("gates and tokens must have the same dtype")
    cdt = compute_dtype(gates.dtype)
    if initial_state is not None:
        assert initial_state.shape == (B, C)
    if T == 0:
        return torch.zeros(B, C, dtype=cdt, device=gates.device) if initial_state is None else initial_state.to(cdt)
    with torch.no_grad():
        carry = torch.empty(B * C, 2, dtype=cdt, device=gates.device)
        _native.reduce_forward(gates, tokens, carry)
        prod, state = carry[:, 0].reshape(B, C), carry[:, 1].reshape(B, C)
        if initial_state is not None:
            state = prod * initial_state.to(cdt) + state
    return state
