"""Generate the golden vectors under tests/golden/ from the reference itself.

Run where the reference checkout is present:

    python tests/golden/make_golden.py path/to/reference

It loads the reference's oracle module accelerated_scan/ref.py by file path
(pure torch, runs on CPU), draws the seeded inputs the reference's own tests
use (tests/test_eq.py:9-23,43-62; tests/tests_eq_complex.py:7-52,66-86) on the
CPU generator, and stores inputs, forward outputs and torch-autograd gradients
as small .npz files.  The fixtures pin this repository's CPU oracle and, through
it, the CUDA kernels; the reference is not needed to run the tests.
"""
import importlib.util
import math
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_ref(root):
    path = os.path.join(root, "accelerated_scan", "ref.py")
    spec = importlib.util.spec_from_file_location("reference_ref_scan", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.scan


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().numpy()
        out[k] = v
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: (getattr(v, "shape", None), getattr(v, "dtype", None)) for k, v in out.items()})


def real_case(scan, name, seed, shape, *, gates_kind, loss, reverse=False):
    torch.manual_seed(seed)
    if gates_kind == "uniform":            # tests/test_eq.py:16-19
        gates = torch.rand(*shape)
    else:                                  # tests/bench.py:8 (without the fp16 rounding)
        gates = 0.999 + 0.001 * torch.rand(*shape)
    tokens = torch.rand(*shape)
    gates.requires_grad_(True)
    tokens.requires_grad_(True)
    out = scan(gates, tokens, reverse=reverse)
    arrays = dict(gates=gates, tokens=tokens, out=out, reverse=np.array(int(reverse)))
    if loss == "mean_sum":                 # tests/test_eq.py:49
        out.mean(dim=-1).sum().backward()
        grad_out = torch.full(shape, 1.0 / shape[-1])
    elif loss == "randn":                  # grad_out ~ N(0,1)
        grad_out = torch.randn(*shape)
        out.backward(grad_out)
    else:
        grad_out = None
    if grad_out is not None:
        arrays.update(grad_out=grad_out, d_gates=gates.grad, d_tokens=tokens.grad)
    save(name, **arrays)


def complex_case(scan, name, seed, shape, *, mode, loss):
    torch.manual_seed(seed)
    if mode in ("hard", "easy"):           # tests/tests_eq_complex.py:26-47
        angle = 2 * torch.pi * torch.rand(*shape)
        radius = 0.99 + 0.01 * torch.rand_like(angle) if mode == "hard" else 0.4 + 0.6 * torch.rand_like(angle)
        forget = torch.polar(radius, angle).to(torch.complex64)
        inputs = torch.randn(*shape).tanh()
    else:                                  # r ~ U(0.9, 0.999), theta ~ U(-pi, pi), complex normal tokens
        radius = 0.9 + 0.099 * torch.rand(*shape)
        angle = (2 * torch.rand(*shape) - 1) * math.pi
        forget = torch.polar(radius, angle).to(torch.complex64)
        inputs = torch.complex(torch.randn(*shape), torch.randn(*shape))
    forget.requires_grad_(True)
    inputs.requires_grad_(True)
    out = scan(forget, inputs)
    if loss == "real_mean":                # tests/tests_eq_complex.py:10-11
        val = out.real.mean()
    elif loss == "last_sum":               # tests/tests_eq_complex.py:14-15
        val = out[:, :, -1].real.sum() + out[:, :, -1].imag.sum()
    elif loss == "abs_sq_mean":            # tests/tests_eq_complex.py:18-19
        val = out.abs().square().mean()
    else:
        val = None
    if val is not None:
        # d(loss)/d(out) in torch's convention for complex leaves, recorded so
        # the oracle's backward can be fed the same upstream gradient
        (grad_out,) = torch.autograd.grad(val, out, retain_graph=True)
        val.backward()
    else:
        grad_out = torch.complex(torch.randn(*shape), torch.randn(*shape))
        out.backward(grad_out)
    save(name, forget=forget, inputs=inputs, out=out, grad_out=grad_out,
         d_forget=forget.grad, d_inputs=inputs.grad)


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py path/to/reference   (the checkout that holds accelerated_scan/ref.py)")
    root = sys.argv[1]
    scan = load_ref(root)
    torch.set_num_threads(1)
    # configuration "fp32 forward, (1, 16, 1024), gates 0.999+0.001*U, tokens U, seed 0"
    real_case(scan, "real_cfg1_b1_c16_t1024_seed0", 0, (1, 16, 1024), gates_kind="near_one", loss=None)
    # seeds and input law of tests/test_eq.py, small channel counts
    real_case(scan, "real_seed3407_t32", 3407, (1, 4, 32), gates_kind="uniform", loss="mean_sum")
    real_case(scan, "real_seed4_t1024", 4, (1, 4, 1024), gates_kind="uniform", loss="mean_sum")
    real_case(scan, "real_seed42_t4099", 42, (1, 2, 4099), gates_kind="uniform", loss="randn")
    real_case(scan, "real_seed57_t8000", 57, (1, 2, 8000), gates_kind="near_one", loss="randn")
    real_case(scan, "real_seed1_t100_reverse", 1, (2, 3, 100), gates_kind="uniform", loss=None, reverse=True)
    # seeds, input law and losses of tests/tests_eq_complex.py
    complex_case(scan, "complex_seed1_hard_t4096_real_mean", 1, (1, 1, 4096), mode="hard", loss="real_mean")
    complex_case(scan, "complex_seed11_easy_t1000_last_sum", 11, (1, 2, 1000), mode="easy", loss="last_sum")
    complex_case(scan, "complex_seed22_hard_t2048_abs_sq_mean", 22, (1, 1, 2048), mode="hard", loss="abs_sq_mean")
    complex_case(scan, "complex_cfg4law_t1024_randn", 0, (1, 2, 1024), mode="cfg4", loss=None)


if __name__ == "__main__":
    main()
