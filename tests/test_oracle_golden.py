"""The CPU oracle against the golden vectors made from the reference's ref.py
(tests/golden/make_golden.py).  Runs without a GPU."""
import numpy as np
import pytest

from helpers import golden_files, rel_err
from oracle import scan_oracle


@pytest.mark.parametrize("path", golden_files("real_"))
def test_real_forward_bit_exact(path):
    d = np.load(path)
    out = scan_oracle.scan(d["gates"], d["tokens"], reverse=bool(d["reverse"]))
    assert np.array_equal(out, d["out"])


@pytest.mark.parametrize("path", [p for p in golden_files("real_") if "d_gates" in np.load(p)])
def test_real_backward_matches_autograd(path):
    d = np.load(path)
    dg, dx = scan_oracle.scan_backward(d["gates"], d["out"], d["grad_out"])
    # hand-written backward vs torch autograd through the tree: different rounding order
    assert rel_err(dx, d["d_tokens"]) <= 2e-6
    assert rel_err(dg, d["d_gates"]) <= 2e-6


@pytest.mark.parametrize("path", golden_files("complex_"))
def test_complex_forward_bit_exact(path):
    d = np.load(path)
    out = scan_oracle.scan(d["forget"], d["inputs"])
    assert np.array_equal(out, d["out"])


@pytest.mark.parametrize("path", golden_files("complex_"))
def test_complex_backward_matches_autograd(path):
    d = np.load(path)
    dg, dx = scan_oracle.scan_backward(d["forget"], d["out"], d["grad_out"])
    if not np.iscomplexobj(d["d_inputs"]):
        dx = dx.real                      # real inputs get a real gradient (complex.py:217-218)
    assert rel_err(dx, d["d_inputs"]) <= 2e-6
    assert rel_err(dg, d["d_forget"]) <= 2e-6
    np.testing.assert_allclose(dg, d["d_forget"], atol=1e-5, rtol=1e-4)   # tests_eq_complex.py:23
    np.testing.assert_allclose(dx, d["d_inputs"], atol=1e-5, rtol=1e-4)


def test_backward_identity_known_answer():
    """The relation the reference pins in tests/test_eq.py:65-90: a reverse scan over
    the gates shifted by one step of dL/dx = 1 gives the token gradient; times the
    previous state it gives the gate gradient.  Checked here against the float64
    recurrence differentiated by hand."""
    rng = np.random.default_rng(1)
    T = 257
    f = rng.standard_normal((1, 1, T)).astype(np.float32) * 0.5
    x = rng.standard_normal((1, 1, T)).astype(np.float32)
    c = scan_oracle.scan(f, x)
    dg, dx = scan_oracle.scan_backward(f, c, np.ones_like(c))
    # exact: g[t] = 1 + f[t+1] g[t+1]
    g = np.zeros(T + 1, dtype=np.float64)
    for t in range(T - 1, -1, -1):
        g[t] = 1.0 + (f[0, 0, t + 1] * g[t + 1] if t + 1 < T else 0.0)
    cex = scan_oracle.scan_exact(f, x)[0, 0]
    want_dg = np.concatenate([[0.0], cex[:-1]]) * g[:T]
    assert rel_err(dx[0, 0], g[:T]) <= 1e-5
    assert rel_err(dg[0, 0], want_dg) <= 2e-5


def test_tree_vs_exact_recurrence():
    rng = np.random.default_rng(0)
    for T in (1, 2, 3, 31, 32, 33, 1000, 4096):
        g = rng.random((2, 2, T), dtype=np.float32)
        x = rng.random((2, 2, T), dtype=np.float32)
        for rev in (False, True):
            assert rel_err(scan_oracle.scan(g, x, reverse=rev), scan_oracle.scan_exact(g, x, reverse=rev)) <= 1e-6
