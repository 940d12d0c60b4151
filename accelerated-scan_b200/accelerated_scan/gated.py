"""Scan with sigmoid gates, the activation fused into the kernels.

    out = scan(gate_logits, tokens)        # x[t] = sigmoid(gate_logits[t]) * x[t-1] + tokens[t]

The reference takes ready-made gates (warp.py:68-83), so a model whose gates are
`sigmoid(z)` pays an elementwise pass over the (B, C, T) tensors before the scan and another
one in the backward.  Here the forward kernel reads the logits and the fused backward
returns the gradient of the logits directly: per element 3 values move in the forward and 5
in the backward, as in the plain scan, instead of 5 and 8.  The sigmoid is evaluated in
fp32 inside the kernels and is never rounded to the storage dtype.

Shapes or alignments without a fused kernel (rows shorter than a few tiles, unaligned
storage offsets) keep the same arithmetic with separate passes: sigmoid and scan in fp32,
results rounded once to the storage dtype.
"""
import torch

from . import _native


class SigmoidGateScan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_logits, tokens):
        B, C, T = gate_logits.shape
        assert tokens.shape == (B, C, T)
        assert gate_logits.is_contiguous()
        assert tokens.is_contiguous()
        if gate_logits.dtype != tokens.dtype:
            raise RuntimeError("gate_logits and tokens must have the same dtype")
        if gate_logits.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            raise RuntimeError(f"unsupported dtype {gate_logits.dtype}")
        states = torch.empty_like(tokens)
        if states.numel() and not _native.forward_sigmoid_gates(gate_logits, tokens, states):
            gates = torch.sigmoid(gate_logits.float())
            if states.dtype == torch.float32:
                _native.forward(gates, tokens, states)
            else:
                wide = torch.empty_like(gates)
                _native.forward(gates, tokens.float(), wide)
                states.copy_(wide)
        ctx.save_for_backward(gate_logits, states)
        return states

    @staticmethod
    def backward(ctx, grad_output):
        gate_logits, states = ctx.saved_tensors
        grad_output = grad_output.contiguous()
        d_logits = torch.empty_like(gate_logits)
        d_tokens = torch.empty_like(gate_logits)
        if states.numel() and not _native.backward_sigmoid_gates(gate_logits, states, grad_output, d_logits, d_tokens):
            gates = torch.sigmoid(gate_logits.float())
            d_gates = torch.empty_like(gates)
            wide = torch.empty_like(gates)
            _native.backward(gates, states.float(), grad_output.float(), d_gates, wide)
            d_tokens.copy_(wide)
            d_logits.copy_(d_gates * (gates * (1.0 - gates)))
        return d_logits, d_tokens


def scan(gate_logits, tokens):
    """Solve x[t] = sigmoid(gate_logits[t]) * x[t-1] + tokens[t].

    Arguments:
        gate_logits (torch.Tensor): shape (B, C, T), CUDA, contiguous; float32, bfloat16 or float16.
        tokens (torch.Tensor): same shape and dtype.

    Returns:
        (torch.Tensor): shape (B, C, T)
    """
    return SigmoidGateScan.apply(gate_logits, tokens)
