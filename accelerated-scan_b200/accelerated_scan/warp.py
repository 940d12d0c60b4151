"""Drop-in replacement of the reference module accelerated_scan/warp.py.

Same names, argument meaning and error behaviour: `scan`, `Scan`, `scan_forward`,
`warpscan_forward`, `warpscan_backward` (reference warp.py:29-83).  The native side
is the prebuilt C-ABI library (include/ascan_b200.h) instead of a JIT-built pybind
module.  Beyond the reference's domain (power-of-two T from 32 to 65536, warp.cuh:379)
any T >= 1 is accepted; bf16/fp16 accumulate in fp32.
"""
import torch

from . import _native


def _check_same(*tensors):
    first = tensors[0]
    for t in tensors[1:]:
        if t.dtype != first.dtype:
            raise RuntimeError("all tensors must have the same dtype")       # warp.cuh:400-401,414-417
        if t.shape != first.shape:
            raise RuntimeError("all tensors must have the same shape")       # warp.cuh:418-421
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError("tensors must be CUDA tensors")               # warp.cuh:396-397
        if not t.is_contiguous():
            raise RuntimeError("tensors must be contiguous")                 # warp.cuh:398-399
        if t.dim() != 3:
            raise RuntimeError("tensors must have shape (B, C, T)")


def warpscan_forward(gates, tokens, out, reverse=False):
    """out[t] = gates[t]*out[t-1] + tokens[t] (from the last step when `reverse`).
    Writes into and returns `out` (reference warp.cuh:394-405)."""
    _check_same(gates, tokens, out)
    if gates.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise RuntimeError(f"unsupported dtype {gates.dtype}")                # warp.cuh:391
    if gates.numel():
        _native.forward(gates, tokens, out, reverse=reverse)
    return out


def warpscan_backward(gates, output, outGrad, gateGradOut, tokenGradOut):
    """Fused backward: fills gateGradOut and tokenGradOut from the saved forward
    output and the output gradient (reference warp.cuh:407-424)."""
    _check_same(gates, output, outGrad, gateGradOut, tokenGradOut)
    if gates.dtype not in (torch.float32, torch.bfloat16, torch.float16):
        raise RuntimeError(f"unsupported dtype {gates.dtype}")
    if gates.numel():
        _native.backward(gates, output, outGrad, gateGradOut, tokenGradOut)


def scan_forward(gates, tokens, reverse=False):
    """Allocates the output and runs the forward kernel (reference warp.py:32-35;
    the output is not zero-filled first, the kernel writes every element)."""
    output = torch.empty_like(tokens)
    warpscan_forward(gates, tokens, output, reverse)
    return output


class Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, tokens):
        B, C, T = gates.shape
        assert tokens.shape == (B, C, T)
        assert gates.is_contiguous()
        assert tokens.is_contiguous()

        states = scan_forward(gates, tokens)
        ctx.save_for_backward(states, gates)
        return states

    # the backward is a reverse scan over the gates shifted by one step
    # (reference warp.py:50-65)
    @staticmethod
    def backward(ctx, grad_output):
        states, gates = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        assert states.is_contiguous()
        assert gates.is_contiguous()

        d_gates = torch.empty_like(gates)
        d_tokens = torch.empty_like(gates)
        warpscan_backward(gates, states, grad_output, d_gates, d_tokens)
        return d_gates, d_tokens


def scan(gates, tokens):
    """Solve the first-order recurrence x[t] = gates[t] * x[t-1] + tokens[t].

    Arguments:
        gates (torch.Tensor): shape (B, C, T), CUDA, contiguous; float32, bfloat16 or float16.
        tokens (torch.Tensor): same shape and dtype.

    Returns:
        (torch.Tensor): shape (B, C, T)
    """
    return Scan.apply(gates, tokens)
