"""The exchange logic of the time-sharded scan on CPU ranks (gloo, world_size 2 and 3):
carry all_gather, prefix/suffix folds, halo plumbing.  The local steps are injected
(straight loops in float64), so no GPU is needed; results are compared with the CPU
oracle on the unsharded sequence.  Also: fold algebra and a rank that fails."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from accelerated_scan import sharded
from oracle import scan_oracle


class LoopOps:
    """Local steps of sharded.NativeOps restated as plain loops (test double)."""

    @staticmethod
    def _rows(t):
        return t.reshape(-1, t.shape[-1])

    fold = staticmethod(sharded.fold_with_tensor_ops)

    @staticmethod
    def reduce_forward(gates, tokens, payload):
        a, b = LoopOps._rows(gates).to(torch.complex128), LoopOps._rows(tokens).to(torch.complex128)
        P = torch.ones(a.shape[0], dtype=a.dtype)
        S = torch.zeros(a.shape[0], dtype=a.dtype)
        for t in range(a.shape[1]):
            S = a[:, t] * S + b[:, t]
            P = P * a[:, t]
        cdt = sharded.compute_dtype(gates.dtype)
        conv = (lambda z: z.to(cdt)) if cdt.is_complex else (lambda z: z.real.to(cdt))
        payload[:, 0] = conv(P)
        payload[:, 1] = conv(S)

    @staticmethod
    def forward(gates, tokens, carry_in):
        a, b = LoopOps._rows(gates).to(torch.complex128), LoopOps._rows(tokens).to(torch.complex128)
        x = torch.zeros(a.shape[0], dtype=a.dtype) if carry_in is None else carry_in.to(torch.complex128)
        out = torch.empty_like(a)
        for t in range(a.shape[1]):
            x = a[:, t] * x + b[:, t]
            out[:, t] = x
        out = out if gates.dtype.is_complex else out.real
        return out.to(gates.dtype).reshape(gates.shape)

    @staticmethod
    def reduce_backward(gates, grad_out, halo_gate_right, payload):
        a, go = LoopOps._rows(gates).to(torch.complex128), LoopOps._rows(grad_out).to(torch.complex128)
        T = a.shape[1]
        nxt = torch.ones(a.shape[0], dtype=a.dtype) if halo_gate_right is None else halo_gate_right.to(torch.complex128)
        P = torch.ones(a.shape[0], dtype=a.dtype)
        g = torch.zeros(a.shape[0], dtype=a.dtype)
        for t in range(T - 1, -1, -1):
            an = torch.conj(a[:, t + 1]) if t + 1 < T else torch.conj(nxt)
            g = an * g + go[:, t]
            P = P * an
        cdt = sharded.compute_dtype(gates.dtype)
        conv = (lambda z: z.to(cdt)) if cdt.is_complex else (lambda z: z.real.to(cdt))
        payload[:, 0] = conv(P)
        payload[:, 1] = conv(g)

    @staticmethod
    def backward(gates, states, grad_out, carry_in, halo_gate_right, halo_state_left):
        a = LoopOps._rows(gates).to(torch.complex128)
        x = LoopOps._rows(states).to(torch.complex128)
        go = LoopOps._rows(grad_out).to(torch.complex128)
        R, T = a.shape
        nxt = torch.ones(R, dtype=a.dtype) if halo_gate_right is None else halo_gate_right.to(torch.complex128)
        g = torch.zeros(R, dtype=a.dtype) if carry_in is None else carry_in.to(torch.complex128)
        xl = torch.zeros(R, dtype=a.dtype) if halo_state_left is None else halo_state_left.to(torch.complex128)
        d_tokens = torch.empty_like(a)
        d_gates = torch.empty_like(a)
        for t in range(T - 1, -1, -1):
            an = torch.conj(a[:, t + 1]) if t + 1 < T else torch.conj(nxt)
            g = an * g + go[:, t]
            d_tokens[:, t] = g
            xp = x[:, t - 1] if t > 0 else xl
            d_gates[:, t] = torch.conj(xp) * g
        if not gates.dtype.is_complex:
            d_gates, d_tokens = d_gates.real, d_tokens.real
        return d_gates.to(gates.dtype).reshape(gates.shape), d_tokens.to(gates.dtype).reshape(gates.shape)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(cplx, shape, seed=5):
    g = torch.Generator().manual_seed(seed)
    if cplx:
        gates = torch.polar(0.8 + 0.19 * torch.rand(*shape, generator=g), 6.28 * torch.rand(*shape, generator=g))
        tokens = torch.complex(torch.randn(*shape, generator=g), torch.randn(*shape, generator=g))
        grad = torch.complex(torch.randn(*shape, generator=g), torch.randn(*shape, generator=g))
    else:
        gates = 0.5 + 0.5 * torch.rand(*shape, generator=g)
        tokens = torch.rand(*shape, generator=g)
        grad = torch.randn(*shape, generator=g)
    return gates, tokens, grad


def _worker(rank, world, port, cplx, fail_rank, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        shape = (2, 3, 60)
        gates, tokens, grad = _inputs(cplx, shape)
        gl, xl, gol = (sharded.shard_time(t, rank, world) for t in (gates, tokens, grad))
        if rank == fail_rank:
            raise RuntimeError("injected failure before the exchange")
        states, carry_in, halo = sharded.time_sharded_forward(gl, xl, None, ops=LoopOps)
        d_gates, d_tokens = sharded.time_sharded_backward(gl, states, gol, carry_in, halo, None, ops=LoopOps)
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), states=states.numpy(), d_gates=d_gates.numpy(),
                 d_tokens=d_tokens.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("cplx", [False, True])
def test_time_sharded_exchange_gloo(tmp_path, world, cplx):
    port = _free_port()
    mp.spawn(_worker, args=(world, port, cplx, -1, str(tmp_path)), nprocs=world, join=True)
    gates, tokens, grad = _inputs(cplx, (2, 3, 60))
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad.numpy())
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    got = np.concatenate([p["states"] for p in parts], axis=-1)
    got_dg = np.concatenate([p["d_gates"] for p in parts], axis=-1)
    got_dx = np.concatenate([p["d_tokens"] for p in parts], axis=-1)
    for a, b in ((got, want), (got_dg, want_dg), (got_dx, want_dx)):
        assert np.abs(a - b).max() / np.abs(b).max() <= 1e-5


def test_rank_failure_surfaces_on_host(tmp_path):
    """A rank that raises before the exchange: the others do not hang, their collective
    ends with an error within the process-group timeout, and the launcher sees it."""
    port = _free_port()
    with pytest.raises(Exception):
        mp.spawn(_worker, args=(2, port, False, 1, str(tmp_path)), nprocs=2, join=True)
    assert not (tmp_path / "rank1.npz").exists()


def test_fold_algebra():
    g = torch.Generator().manual_seed(0)
    world, rows = 5, 7
    P = torch.rand(world, rows, generator=g)
    S = torch.randn(world, rows, generator=g)
    x = torch.zeros(rows)
    for k in range(world):
        assert torch.allclose(sharded.fold_prefix(P, S, k), x)
        x = P[k] * x + S[k]
    gsuf = torch.zeros(rows)
    for k in range(world - 1, -1, -1):
        assert torch.allclose(sharded.fold_suffix(P, S, k), gsuf)
        gsuf = P[k] * gsuf + S[k]


def test_shard_helpers():
    t = torch.arange(2 * 3 * 10, dtype=torch.float32).reshape(2, 3, 10)
    assert torch.equal(torch.cat([sharded.shard_time(t, r, 3) for r in range(3)], dim=-1), t)
    rows = torch.cat([sharded.shard_rows(t, r, 4) for r in range(4)], dim=1)
    assert torch.equal(rows.reshape(2, 3, 10), t)
    assert sharded.compute_dtype(torch.bfloat16) == torch.float32
    assert sharded.compute_dtype(torch.complex64) == torch.complex64
