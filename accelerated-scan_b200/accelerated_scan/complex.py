"""Drop-in replacement of the reference module accelerated_scan/complex.py.

`scan(forget, inputs)` and `Scan` keep the reference's behaviour (complex.py:157-239):
`forget` must be complex, real `inputs` are treated as complex with a zero imaginary
part and their gradient is returned real.  The two Triton kernels are replaced by the
hand-written CUDA kernels behind the C ABI; `forward_scan` / `backward_scan` keep the
`kernel[grid](...)` call form that the reference's benchmark uses
(tests/bench_complex.py:4,31-45).
"""
import torch

from . import _native


class _GridLaunch:
    """Mimics the `kernel[(B, C)](...)` call form of the Triton kernels.  The grid is
    ignored: the library plans its own launch."""

    def __init__(self, fn):
        self._fn = fn

    def __getitem__(self, grid):
        return self._fn


def _as_complex(real_view):
    return torch.view_as_complex(real_view)


def _forward_scan(forget_real, inputs_real, states_real, seqlen=None, **_ignored):
    # arguments are view_as_real tensors of shape (B, C, T, 2), as in complex.py:174-180
    _native.forward(_as_complex(forget_real), _as_complex(inputs_real), _as_complex(states_real))


def _backward_scan(forget_real, states_real, d_output_real, d_inputs_real, d_forget_real, seqlen=None, **_ignored):
    # argument order of complex.py:205-213
    _native.backward(_as_complex(forget_real), _as_complex(states_real), _as_complex(d_output_real),
                     _as_complex(d_forget_real), _as_complex(d_inputs_real))


forward_scan = _GridLaunch(_forward_scan)
backward_scan = _GridLaunch(_backward_scan)


class Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, forget, inputs):
        if not torch.is_complex(forget):
            raise TypeError("forget must be a complex tensor")
        if forget.dtype != torch.complex64:
            raise RuntimeError("forget must be complex64")
        real_inputs = not torch.is_complex(inputs)
        inputs_dtype = inputs.dtype
        B, C, T = forget.shape
        assert inputs.shape == (B, C, T)
        assert forget.is_contiguous()
        assert inputs.is_contiguous()

        if not real_inputs and inputs.dtype != torch.complex64:
            raise RuntimeError("inputs must be complex64 or real")

        states = torch.empty_like(forget)
        fused = False
        if real_inputs and states.numel() and inputs.dtype == torch.float32:
            # real tokens go straight into the kernel (no complex copy of the inputs) ...
            fused = _native.forward_complex_real_tokens(forget, inputs, states)
        if not fused:
            # ... unless the shape has no fused kernel: promote as the reference does (complex.py:168-169)
            if real_inputs:
                inputs = torch.complex(inputs.float(), torch.zeros_like(inputs, dtype=torch.float32))
            if states.numel():
                _native.forward(forget, inputs, states)
        ctx.save_for_backward(forget, states)
        ctx.real_inputs = real_inputs
        ctx.inputs_dtype = inputs_dtype
        return states

    # reverse scan over the conjugated gates shifted by one step (complex.py:188-219)
    @staticmethod
    def backward(ctx, d_output):
        forget, states = ctx.saved_tensors
        d_output = d_output.contiguous()
        assert forget.is_contiguous()
        assert states.is_contiguous()

        d_forget = torch.empty_like(forget)
        if ctx.real_inputs and states.numel():
            # real inputs: the kernel writes the real part of their gradient only (complex.py:217-218)
            d_real = torch.empty(states.shape, dtype=torch.float32, device=states.device)
            if _native.backward_complex_real_tokens(forget, states, d_output, d_forget, d_real):
                return d_forget, d_real.to(ctx.inputs_dtype)
        d_inputs = torch.empty_like(states)
        if states.numel():
            _native.backward(forget, states, d_output, d_forget, d_inputs)
        if ctx.real_inputs:
            d_inputs = d_inputs.real.to(ctx.inputs_dtype)
        return d_forget, d_inputs


def scan(forget, inputs):
    """Solve x[t] = forget[t] * x[t-1] + inputs[t] with complex coefficients.

    Arguments:
        forget (torch.Tensor): shape (B, C, T), complex64, CUDA, contiguous.  Any T.
        inputs (torch.Tensor): shape (B, C, T), complex64 or real (imaginary part zero).

    Returns:
        (torch.Tensor): complex64, same shape as inputs
    """
    return Scan.apply(forget, inputs)
