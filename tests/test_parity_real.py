"""CUDA kernels (through the drop-in Python API and the C ABI) against the CPU
oracle on the same seeded inputs: real dtypes.  Mirrors the reference's
tests/test_eq.py (seeds, shapes, input law, tolerances) with the inputs drawn on
the CPU generator."""
import numpy as np
import pytest
import torch

from helpers import golden_files, real_inputs, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

SEEDS = [3407, 4, 42, 57]                                      # reference tests/test_eq.py:9
SEQLENS = [2 ** i for i in range(5, 17)] + [16323, 8000, 33753, 127323]   # test_eq.py:10
FP32_REL = 1e-5            # max|err| / max|ref|, forward and backward
BF16_REL = 2.0 ** -8       # vs the oracle evaluated in fp32 on the bf16-rounded inputs
F16_REL = 2.0 ** -10


def _warp():
    import accelerated_scan.warp as warp
    return warp


@pytest.mark.parametrize("path", golden_files("real_"))
def test_golden_vectors(cuda_device, path):
    warp = _warp()
    d = np.load(path)
    gates = torch.from_numpy(d["gates"]).to(cuda_device)
    tokens = torch.from_numpy(d["tokens"]).to(cuda_device)
    if bool(d["reverse"]):
        out = warp.scan_forward(gates, tokens, reverse=True)
    else:
        gates.requires_grad_(True)
        tokens.requires_grad_(True)
        out = warp.scan(gates, tokens)
    assert rel_err(to_np(out), d["out"]) <= FP32_REL
    torch.testing.assert_close(out.detach().cpu(), torch.from_numpy(d["out"]), atol=2e-6, rtol=1e-5)
    if "d_gates" in d:
        out.backward(torch.from_numpy(d["grad_out"]).to(cuda_device))
        assert rel_err(to_np(gates.grad), d["d_gates"]) <= FP32_REL
        assert rel_err(to_np(tokens.grad), d["d_tokens"]) <= FP32_REL


@pytest.mark.parametrize("seed", SEEDS[:2])
@pytest.mark.parametrize("seqlen", SEQLENS)
def test_fp32_forward_backward(cuda_device, seed, seqlen):
    """test_eq_forward / test_eq_backward of the reference, shape (1, 512, T) cut to
    64 channels so the CPU oracle stays fast."""
    warp = _warp()
    shape = (1, 64, seqlen)
    gates, tokens, grad_out = real_inputs(seed, shape)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad_out.numpy())
    g = gates.to(cuda_device).requires_grad_(True)
    x = tokens.to(cuda_device).requires_grad_(True)
    out = warp.scan(g, x)
    out.backward(grad_out.to(cuda_device))
    assert rel_err(to_np(out), want) <= FP32_REL
    assert rel_err(to_np(x.grad), want_dx) <= FP32_REL
    assert rel_err(to_np(g.grad), want_dg) <= FP32_REL


@pytest.mark.parametrize("seqlen", [32, 100, 1024, 4099, 65536])
def test_fp32_mean_sum_loss(cuda_device, seqlen):
    """The reference's backward test loss: scan(...).mean(dim=-1).sum() (test_eq.py:49)."""
    warp = _warp()
    gates, tokens, _ = real_inputs(42, (1, 32, seqlen), grad=False)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    go = np.full_like(want, 1.0 / seqlen)
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, go)
    g = gates.to(cuda_device).requires_grad_(True)
    x = tokens.to(cuda_device).requires_grad_(True)
    warp.scan(g, x).mean(dim=-1).sum().backward()
    assert rel_err(to_np(x.grad), want_dx) <= FP32_REL
    assert rel_err(to_np(g.grad), want_dg) <= FP32_REL


@pytest.mark.parametrize("seqlen", [1, 2, 3, 5, 31, 33, 95, 96, 97, 383, 384, 385, 767, 768, 769, 1000, 1537, 3001])
@pytest.mark.parametrize("rows", [(1, 1), (1, 5), (3, 7)])
def test_fp32_small_and_ragged(cuda_device, seqlen, rows):
    """Every tile/row-boundary alignment: T around the tile sizes, few rows, T that
    is not a multiple of 16 bytes (plain loader) and T that is."""
    warp = _warp()
    shape = (rows[0], rows[1], seqlen)
    gates, tokens, grad_out = real_inputs(7, shape)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_rev = scan_oracle.scan(gates.numpy(), tokens.numpy(), reverse=True)
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad_out.numpy())
    g, x = gates.to(cuda_device), tokens.to(cuda_device)
    out = warp.scan_forward(g, x)
    rev = warp.scan_forward(g, x, reverse=True)
    dg, dx = torch.empty_like(g), torch.empty_like(g)
    warp.warpscan_backward(g, out, grad_out.to(cuda_device), dg, dx)
    assert rel_err(to_np(out), want) <= FP32_REL
    assert rel_err(to_np(rev), want_rev) <= FP32_REL
    assert rel_err(to_np(dx), want_dx) <= FP32_REL
    assert rel_err(to_np(dg), want_dg) <= FP32_REL


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, BF16_REL), (torch.float16, F16_REL)])
@pytest.mark.parametrize("seqlen", [32, 128, 1024, 4096, 8000, 16323, 65536])
@pytest.mark.parametrize("law", ["uniform", "near_one"])
def test_half_precision_fp32_accumulation(cuda_device, dtype, tol, seqlen, law):
    """16-bit storage, fp32 accumulation: compared with the oracle evaluated in fp32
    on the rounded inputs; the only error left is the final rounding of each output."""
    warp = _warp()
    if dtype == torch.float16 and law == "near_one" and seqlen > 1024:
        pytest.skip("states and gate gradients exceed the fp16 range")
    shape = (1, 32, seqlen)
    gates, tokens, grad_out = real_inputs(3407, shape, law=law, dtype=dtype)
    gf, xf, gof = gates.float().numpy(), tokens.float().numpy(), grad_out.float().numpy()
    want = scan_oracle.scan(gf, xf)
    g = gates.to(cuda_device).requires_grad_(True)
    x = tokens.to(cuda_device).requires_grad_(True)
    out = warp.scan(g, x)
    assert out.dtype == dtype
    assert rel_err(to_np(out), want) <= tol
    # the backward consumes the rounded saved states, as the kernel does
    states = out.detach().float().cpu().numpy()
    want_dg, want_dx = scan_oracle.scan_backward(gf, states, gof)
    out.backward(grad_out.to(cuda_device))
    assert rel_err(to_np(x.grad), want_dx) <= tol
    assert rel_err(to_np(g.grad), want_dg) <= tol


def test_reference_config_1(cuda_device):
    """fp32 forward, (1, 16, 1024), gates 0.999 + 0.001*U, tokens U, seed 0, elementwise."""
    warp = _warp()
    gates, tokens, _ = real_inputs(0, (1, 16, 1024), law="near_one", grad=False)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    out = warp.scan(gates.to(cuda_device), tokens.to(cuda_device))
    np.testing.assert_allclose(to_np(out), want, rtol=1e-5, atol=0)


def test_reference_config_2(cuda_device):
    """fp32 forward+backward, (8, 1536, 4096), U(0,1) gates/tokens, N(0,1) grad_out;
    out, grad_gates and grad_tokens within 1e-5 relative."""
    warp = _warp()
    gates, tokens, grad_out = real_inputs(0, (8, 1536, 4096))
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad_out.numpy())
    g = gates.to(cuda_device).requires_grad_(True)
    x = tokens.to(cuda_device).requires_grad_(True)
    out = warp.scan(g, x)
    out.backward(grad_out.to(cuda_device))
    assert rel_err(to_np(out), want) <= FP32_REL
    assert rel_err(to_np(x.grad), want_dx) <= FP32_REL
    assert rel_err(to_np(g.grad), want_dg) <= FP32_REL


def test_unaligned_views_use_plain_loader(cuda_device):
    """Pointers that are not 16-byte aligned (a storage offset of one element)."""
    warp = _warp()
    T = 1000
    gates, tokens, grad_out = real_inputs(11, (2, 3, T))
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad_out.numpy())

    def offset(t):
        buf = torch.empty(t.numel() + 1, device=cuda_device, dtype=t.dtype)
        view = buf[1:].view(t.shape)
        view.copy_(t)
        assert view.data_ptr() % 16 != 0 and view.is_contiguous()
        return view

    g, x, go = offset(gates), offset(tokens), offset(grad_out)
    out = offset(torch.zeros_like(gates))
    warp.warpscan_forward(g, x, out, False)
    dg, dx = offset(torch.zeros_like(gates)), offset(torch.zeros_like(gates))
    warp.warpscan_backward(g, out, go, dg, dx)
    assert rel_err(to_np(out), want) <= FP32_REL
    assert rel_err(to_np(dx), want_dx) <= FP32_REL
    assert rel_err(to_np(dg), want_dg) <= FP32_REL


# one shape per launch plan: (rows, seqlen, plan kernel, row_grid)
DETERMINISM_CASES = [
    (7200, 13000, 0, 0),     # chained stream plan, rows split into segments
    (1024, 16384, 2, 0),     # team plan
    (16, 1 << 18, 1, 0),     # look-back plan: segments of a row scanned concurrently by many CTAs
    (12288, 256, 0, 1),      # short rows on the tile grid
]


@pytest.mark.parametrize("rows,seqlen,kernel,row_grid", DETERMINISM_CASES)
def test_deterministic(cuda_device, rows, seqlen, kernel, row_grid):
    """Every plan is bitwise reproducible from run to run, forward and backward: the order in
    which partial results are combined is fixed by the plan (the look-back plan reads the
    aggregates of fixed sets of segments, never "whatever is there"), not by timing.  The
    reference's kernels are deterministic too (one block per row, warp.cuh:49-223)."""
    from accelerated_scan import _native

    pl = _native.plan(rows, seqlen, _native.F32, _native.KIND_FORWARD)
    assert pl["kernel"] == kernel and pl["row_grid"] == row_grid, pl
    gates, tokens, grad_out = real_inputs(5, (1, rows, seqlen), law="near_one")
    g, x, go = gates.to(cuda_device), tokens.to(cuda_device), grad_out.to(cuda_device)
    runs = []
    for _ in range(3):
        out, dg, dx = torch.empty_like(x), torch.empty_like(x), torch.empty_like(x)
        _native.forward(g, x, out)
        _native.backward(g, out, go, dg, dx)
        runs.append((out, dg, dx))
    for other in runs[1:]:
        for a, b in zip(runs[0], other):
            assert torch.equal(a, b)


def test_status_word_clean(cuda_device):
    from accelerated_scan import _native
    _native.check_status(cuda_device)


def test_more_than_2_31_elements(cuda_device):
    """64-bit offsets: a matrix of 2.2e9 elements (the reference indexes with 32-bit ints,
    warp.cuh:58-59).  Rows are independent, so a few rows spread over the matrix are checked
    against the oracle; the inputs are drawn on the GPU and the checked rows copied back."""
    warp = _warp()
    rows, T = 2112, 1 << 20
    assert rows * T > 2 ** 31
    free, _ = torch.cuda.mem_get_info(cuda_device)
    if free < 40 * 2 ** 30:
        pytest.skip("needs about 27 GB of device memory")
    gen = torch.Generator(device=cuda_device).manual_seed(5)
    gates = (0.999 + 0.001 * torch.rand(1, rows, T, device=cuda_device, generator=gen)).to(torch.bfloat16)
    tokens = torch.rand(1, rows, T, device=cuda_device, generator=gen).to(torch.bfloat16)
    grad_out = torch.randn(1, rows, T, device=cuda_device, generator=gen).to(torch.bfloat16)
    out = warp.scan_forward(gates, tokens)
    d_gates, d_tokens = torch.empty_like(gates), torch.empty_like(gates)
    warp.warpscan_backward(gates, out, grad_out, d_gates, d_tokens)
    pick = [0, 1, rows // 2, rows - 2, rows - 1]
    sel = lambda t: t[:, pick].float().cpu().numpy()
    want = scan_oracle.scan(sel(gates), sel(tokens))
    assert rel_err(sel(out), want) <= BF16_REL
    want_dg, want_dx = scan_oracle.scan_backward(sel(gates), sel(out), sel(grad_out))
    assert rel_err(sel(d_tokens), want_dx) <= BF16_REL
    assert rel_err(sel(d_gates), want_dg) <= BF16_REL
