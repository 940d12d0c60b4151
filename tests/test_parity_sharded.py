"""The time-sharded scan on the GPU: the single-pass path (every rank streams its slice once
and takes its incoming state from slice aggregates stored into its exchange buffer) and the
three-step path (carry-only reduction, all_gather, seeded scan).

On one GPU the ranks are emulated one after the other, in the order of their dependencies
(kernels that wait for one another never run side by side on one GPU), and the concatenation
is compared with the CPU oracle on the unsharded sequence.  With two or more GPUs the real
multi-process paths run as child processes."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from helpers import complex_inputs, real_inputs, rel_err, to_np
from oracle import scan_oracle

pytestmark = pytest.mark.gpu

REL = {torch.float32: 1e-5, torch.complex64: 1e-5, torch.bfloat16: 2.0 ** -8}


def _emulate(gates, tokens, grad_out, world, dev):
    from accelerated_scan import sharded

    ops = sharded.NativeOps
    T = gates.shape[-1]
    cuts = [T * r // world for r in range(world + 1)]
    sl = lambda t, r: t[..., cuts[r]:cuts[r + 1]].contiguous().to(dev)
    g = [sl(gates, r) for r in range(world)]
    x = [sl(tokens, r) for r in range(world)]
    go = [sl(grad_out, r) for r in range(world)]
    rows = gates.shape[0] * gates.shape[1]
    cdt = sharded.compute_dtype(gates.dtype)
    # forward: reduce -> (gather) -> fold kernel -> seeded scan
    fwd_payload = []
    for r in range(world):
        pay = torch.empty(rows, 3, dtype=cdt, device=dev)
        ops.reduce_forward(g[r], x[r], pay)
        pay[:, 2] = g[r].reshape(rows, -1)[:, 0]
        fwd_payload.append(pay)
    gathered = torch.stack(fwd_payload)                                   # what all_gather would return
    P, S = gathered[:, :, 0], gathered[:, :, 1]
    cin, halo = [], []
    for r in range(world):
        c, h = ops.fold(gathered, r, False, True)
        # the fold kernel against the plain tensor arithmetic
        c2, h2 = sharded.fold_with_tensor_ops(gathered, r, False, True)
        torch.testing.assert_close(c, c2, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(h, h2)
        cin.append(c)
        halo.append(h)
    states = [ops.forward(g[r], x[r], cin[r] if r > 0 else None) for r in range(world)]
    # backward: reduce -> (gather) -> fold kernel -> seeded fused backward
    bwd_payload = []
    for r in range(world):
        pay = torch.empty(rows, 2, dtype=cdt, device=dev)
        ops.reduce_backward(g[r], go[r], halo[r], pay)
        bwd_payload.append(pay)
    gathered_b = torch.stack(bwd_payload)
    gin = []
    for r in range(world):
        c, _ = ops.fold(gathered_b, r, True, False)
        c2, _ = sharded.fold_with_tensor_ops(gathered_b, r, True, False)
        torch.testing.assert_close(c, c2, rtol=1e-5, atol=1e-6)
        gin.append(c)
    grads = [ops.backward(g[r], states[r], go[r], gin[r], halo[r], cin[r]) for r in range(world)]
    cat = lambda parts: torch.cat(parts, dim=-1)
    return cat(states), cat([d[0] for d in grads]), cat([d[1] for d in grads]), (P, S)


@pytest.mark.parametrize("world", [2, 3, 8])
@pytest.mark.parametrize("seqlen", [96, 1000, 24576, 100000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64, torch.bfloat16])
def test_emulated_time_shards(cuda_device, world, seqlen, dtype):
    shape = (2, 5, seqlen)
    if dtype == torch.complex64:
        gates, tokens, grad_out = complex_inputs(9, shape, law="cfg4")
    else:
        gates, tokens, grad_out = real_inputs(9, shape, law="near_one", dtype=dtype)
    up = (lambda t: t.numpy()) if dtype != torch.bfloat16 else (lambda t: t.float().numpy())
    want = scan_oracle.scan(up(gates), up(tokens))
    states, d_gates, d_tokens, (P, S) = _emulate(gates, tokens, grad_out, world, cuda_device)
    tol = REL[dtype]
    assert rel_err(to_np(states), want) <= tol
    saved = to_np(states) if dtype == torch.bfloat16 else want
    want_dg, want_dx = scan_oracle.scan_backward(up(gates), saved, up(grad_out))
    assert rel_err(to_np(d_tokens), want_dx) <= tol
    assert rel_err(to_np(d_gates), want_dg) <= tol
    # the carries themselves: the product of the gates and the zero-start end state of slice 0
    cut = seqlen // world
    first = scan_oracle.scan(up(gates)[..., :cut], up(tokens)[..., :cut])[..., -1].reshape(-1)
    assert rel_err(to_np(S[0]), first) <= 1e-5
    prod = np.prod(up(gates)[..., :cut].astype(np.complex128 if dtype == torch.complex64 else np.float64), axis=-1).reshape(-1)
    np.testing.assert_allclose(to_np(P[0]).astype(prod.dtype), prod, rtol=2e-4, atol=1e-30)


@pytest.mark.parametrize("rows,seqlen", [(300, 24576), (1024, 6000), (2000, 9216), (3700, 3072)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_emulated_time_shards_many_rows(cuda_device, rows, seqlen, dtype):
    """The same with row counts that take the team plan (carry-only kinds included) and the
    chained stream plan."""
    from accelerated_scan import _native

    world = 2
    code = _native.DTYPE_CODE[dtype]
    expect = 2 if rows < 2 * 148 * 12 else 0
    assert _native.plan(rows, seqlen // world, code, _native.KIND_REDUCE_FORWARD)["kernel"] == expect
    assert _native.plan(rows, seqlen // world, code, _native.KIND_REDUCE_BACKWARD)["kernel"] == expect
    shape = (1, rows, seqlen)
    gates, tokens, grad_out = real_inputs(19, shape, law="near_one", dtype=dtype)
    up = (lambda t: t.numpy()) if dtype != torch.bfloat16 else (lambda t: t.float().numpy())
    want = scan_oracle.scan(up(gates), up(tokens))
    states, d_gates, d_tokens, _ = _emulate(gates, tokens, grad_out, world, cuda_device)
    tol = REL[dtype]
    assert rel_err(to_np(states), want) <= tol
    saved = to_np(states) if dtype == torch.bfloat16 else want
    want_dg, want_dx = scan_oracle.scan_backward(up(gates), saved, up(grad_out))
    assert rel_err(to_np(d_tokens), want_dx) <= tol
    # bf16: at a shard boundary d_gates uses the incoming state in fp32 (the folded carry), the
    # oracle the saved state rounded to bf16: one more half-ulp on that element
    assert rel_err(to_np(d_gates), want_dg) <= (2 * tol if dtype == torch.bfloat16 else tol)
    _native.check_status(cuda_device)


def _emulate_single_pass(gates, tokens, grad_out, world, dev, calls=1):
    """`world` ranks on one GPU, one launch per rank and direction: forward in rank order,
    backward in reverse rank order, so every aggregate a launch waits for is already there."""
    from accelerated_scan import _native, sharded

    T = gates.shape[-1]
    assert T % world == 0
    sl = lambda t, r: t[..., r * (T // world):(r + 1) * (T // world)].contiguous().to(dev)
    g = [sl(gates, r) for r in range(world)]
    x = [sl(tokens, r) for r in range(world)]
    go = [sl(grad_out, r) for r in range(world)]
    rows = gates.shape[0] * gates.shape[1]
    cdt = sharded.compute_dtype(gates.dtype)
    nbytes = _native.exchange_bytes(rows, world)
    fwd_x = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    bwd_x = [torch.zeros(nbytes, dtype=torch.uint8, device=dev) for _ in range(world)]
    fp, bp = [t.data_ptr() for t in fwd_x], [t.data_ptr() for t in bwd_x]
    for call in range(1, calls + 1):
        states = [torch.full_like(x[r], float("nan")) for r in range(world)]
        saved = [torch.full((rows,), float("nan"), dtype=cdt, device=dev) for r in range(world)]
        for r in range(world):
            _native.forward_time_sharded(g[r], x[r], states[r], r, world, call, fp, saved[r])
        dg = [torch.full_like(x[r], float("nan")) for r in range(world)]
        dx = [torch.full_like(x[r], float("nan")) for r in range(world)]
        for r in reversed(range(world)):
            _native.backward_time_sharded(g[r], states[r], go[r], dg[r], dx[r], r, world, call, bp, saved[r])
    _native.check_status(dev)
    cat = lambda parts: torch.cat(parts, dim=-1)
    return cat(states), cat(dg), cat(dx), saved


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("slice_len", [8, 1152, 4104, 40000])
@pytest.mark.parametrize("dtype", [torch.float32, torch.complex64, torch.bfloat16])
def test_single_pass_time_shards_emulated(cuda_device, world, slice_len, dtype):
    shape = (2, 5, slice_len * world)
    if dtype == torch.complex64:
        gates, tokens, grad_out = complex_inputs(9, shape, law="cfg4")
    else:
        gates, tokens, grad_out = real_inputs(9, shape, law="near_one", dtype=dtype)
    up = (lambda t: t.numpy()) if dtype != torch.bfloat16 else (lambda t: t.float().numpy())
    want = scan_oracle.scan(up(gates), up(tokens))
    states, d_gates, d_tokens, saved = _emulate_single_pass(gates, tokens, grad_out, world, cuda_device, calls=3)
    tol = REL[dtype]
    assert rel_err(to_np(states), want) <= tol
    kept = to_np(states) if dtype == torch.bfloat16 else want
    want_dg, want_dx = scan_oracle.scan_backward(up(gates), kept, up(grad_out))
    assert rel_err(to_np(d_tokens), want_dx) <= tol
    assert rel_err(to_np(d_gates), want_dg) <= (2 * tol if dtype == torch.bfloat16 else tol)
    # the state entering every slice is the oracle's state just before it
    for r in range(1, world):
        before = want[..., r * slice_len - 1].reshape(-1)
        assert rel_err(to_np(saved[r]), before) <= max(tol, 1e-5)
    assert float(saved[0].abs().max()) == 0.0


@pytest.mark.parametrize("rows,slice_len,world", [(1024, 6144, 2), (1024, 16384, 8), (300, 9000, 4)])
def test_single_pass_time_shards_many_rows(cuda_device, rows, slice_len, world):
    """Config-5-like row counts (far more rows than SMs), several calls on one set of buffers."""
    shape = (1, rows, slice_len * world)
    gates, tokens, grad_out = real_inputs(23, shape, law="near_one")
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad_out.numpy())
    states, d_gates, d_tokens, _ = _emulate_single_pass(gates, tokens, grad_out, world, cuda_device, calls=4)
    assert rel_err(to_np(states), want) <= 1e-5
    assert rel_err(to_np(d_tokens), want_dx) <= 1e-5
    assert rel_err(to_np(d_gates), want_dg) <= 1e-5


def test_single_pass_partner_never_arrives(cuda_device):
    """Rank 1 of 2 runs although rank 0 never stored its aggregates: every wait gives up after
    its bound, the launch ends, the status reports it, and the next complete run is right."""
    from accelerated_scan import _native, sharded

    rows, slice_len = 64, 8192
    gates, tokens, grad_out = real_inputs(5, (1, rows, 2 * slice_len), law="near_one")
    g1 = gates[..., slice_len:].contiguous().to(cuda_device)
    x1 = tokens[..., slice_len:].contiguous().to(cuda_device)
    xb = [torch.zeros(_native.exchange_bytes(rows, 2), dtype=torch.uint8, device=cuda_device) for _ in range(2)]
    out = torch.empty_like(x1)
    _native.check_status(cuda_device)
    _native.forward_time_sharded(g1, x1, out, 1, 2, 1, [t.data_ptr() for t in xb], None)
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        _native.check_status(cuda_device)
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    states, _, _, _ = _emulate_single_pass(gates, tokens, grad_out, 2, cuda_device)
    assert rel_err(to_np(states), want) <= 1e-5


@pytest.mark.parametrize("seqlen", [7, 100, 3000, 70000])
def test_carry_in_is_initial_state(cuda_device, seqlen):
    """ascan_forward with carry_in continues a scan: scanning [first | second] equals
    scanning `second` from the last state of `first` (streaming / resume use)."""
    from accelerated_scan import _native

    gates, tokens, _ = real_inputs(3, (1, 9, 2 * seqlen), grad=False)
    g, x = gates.to(cuda_device), tokens.to(cuda_device)
    full = torch.empty_like(x)
    _native.forward(g, x, full)
    g2, x2 = g[..., seqlen:].contiguous(), x[..., seqlen:].contiguous()
    cont = torch.empty_like(x2)
    _native.forward(g2, x2, cont, carry_in=full[0, :, seqlen - 1].float().contiguous())
    assert rel_err(to_np(cont), to_np(full[..., seqlen:])) <= 1e-5


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, out_dir, single_pass):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    import datetime
    import torch.distributed as dist
    from accelerated_scan import sharded

    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=60))
    try:
        gates, tokens, grad_out = real_inputs(17, (2, 8, 49152), law="near_one")
        g = sharded.shard_time(gates, rank, world).to(dev).requires_grad_(True)
        x = sharded.shard_time(tokens, rank, world).to(dev).requires_grad_(True)
        go = sharded.shard_time(grad_out, rank, world).to(dev)
        for _ in range(3):                                  # several calls on one set of exchange buffers
            g.grad = x.grad = None
            out = sharded.sharded_scan(g, x, None, dim="time", single_pass=single_pass)
            out.backward(go)
        torch.cuda.synchronize()
        if single_pass:
            from accelerated_scan import _native

            assert sharded.PeerExchange.get(None, 16, dev).usable, "peer exchange could not be set up"
            _native.check_status(dev)
            sharded.PeerExchange.close_all()
        np.savez(os.path.join(out_dir, f"rank{rank}.npz"), states=to_np(out), d_gates=to_np(g.grad),
                 d_tokens=to_np(x.grad))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("single_pass", [True, False])
def test_time_sharded_multi_process(cuda_device, tmp_path, single_pass):
    """One process per GPU: the single-pass path over peer stores, and the three-step path over NCCL."""
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    mp.spawn(_nccl_worker, args=(world, _free_port(), str(tmp_path), single_pass), nprocs=world, join=True)
    gates, tokens, grad_out = real_inputs(17, (2, 8, 49152), law="near_one")
    want = scan_oracle.scan(gates.numpy(), tokens.numpy())
    want_dg, want_dx = scan_oracle.scan_backward(gates.numpy(), want, grad_out.numpy())
    parts = [np.load(tmp_path / f"rank{r}.npz") for r in range(world)]
    cat = lambda k: np.concatenate([p[k] for p in parts], axis=-1)
    assert rel_err(cat("states"), want) <= 1e-5
    assert rel_err(cat("d_tokens"), want_dx) <= 1e-5
    assert rel_err(cat("d_gates"), want_dg) <= 1e-5
