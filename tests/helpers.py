"""Seeded input generators and error metrics shared by the tests.

All random draws use the CPU generator (order: gates, tokens, grad_out) so that the
CPU oracle and the CUDA kernels see identical bits.
"""
import glob
import math
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden_files(prefix):
    return sorted(glob.glob(os.path.join(GOLDEN_DIR, prefix + "*.npz")))


def real_inputs(seed, shape, law="uniform", dtype=torch.float32, grad=True):
    """law 'uniform': gates, tokens ~ U(0,1) (reference tests/test_eq.py:16-19);
    law 'near_one': gates = 0.999 + 0.001*U(0,1) (reference tests/bench.py:8)."""
    g = torch.Generator().manual_seed(seed)
    gates = torch.rand(*shape, generator=g)
    if law == "near_one":
        gates = 0.999 + 0.001 * gates
    tokens = torch.rand(*shape, generator=g)
    grad_out = torch.randn(*shape, generator=g) if grad else None
    cast = lambda t: None if t is None else t.to(dtype)
    return cast(gates), cast(tokens), cast(grad_out)


def complex_inputs(seed, shape, law="hard", real_tokens=False):
    """laws 'hard'/'easy': reference tests/tests_eq_complex.py:26-47;
    'cfg4': r ~ U(0.9, 0.999), theta ~ U(-pi, pi)."""
    g = torch.Generator().manual_seed(seed)
    if law == "cfg4":
        radius = 0.9 + 0.099 * torch.rand(*shape, generator=g)
        angle = (2 * torch.rand(*shape, generator=g) - 1) * math.pi
    else:
        angle = 2 * math.pi * torch.rand(*shape, generator=g)
        u = torch.rand(*shape, generator=g)
        radius = 0.99 + 0.01 * u if law == "hard" else 0.4 + 0.6 * u
    forget = torch.polar(radius, angle).to(torch.complex64)
    if real_tokens:
        inputs = torch.randn(*shape, generator=g).tanh()
    else:
        inputs = torch.complex(torch.randn(*shape, generator=g), torch.randn(*shape, generator=g))
    grad_out = torch.complex(torch.randn(*shape, generator=g), torch.randn(*shape, generator=g))
    return forget, inputs, grad_out


def rel_err(got, want):
    """max|got - want| / max|want| (the relative-to-output-magnitude error)."""
    got = np.asarray(got)
    want = np.asarray(want)
    denom = float(np.abs(want).max())
    if denom == 0.0:
        denom = 1.0
    return float(np.abs(got.astype(want.dtype) - want).max()) / denom


def to_np(t):
    t = t.detach().cpu()
    if t.dtype in (torch.bfloat16, torch.float16):
        t = t.float()
    return t.numpy()
