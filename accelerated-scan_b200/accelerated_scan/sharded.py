"""Multi-GPU sharding of the scan (one process per GPU, `torch.distributed`).

The reference has no multi-device path.  Two ways to shard exist:

* rows (batch x channel): rows are independent, so every rank runs the single-GPU
  scan on its own rows and nothing is exchanged (`shard_rows` only slices).
* time: every rank owns a contiguous time slice of every row.  Two paths:

  single pass (`PeerExchange`, the default where it can be set up): every rank streams its
  slice once with the look-back kernel (`ascan_forward_time_sharded` /
  `ascan_backward_time_sharded`).  The warp that finishes a row's slice stores the slice's
  aggregate, with plain 64-bit peer stores, into the exchange buffers of the later ranks; a
  segment's incoming state is the fold of the earlier ranks' aggregates, read from the
  rank's own buffer, followed by the local look-back.  No collective, no second read.

  three steps (fallback: slices that are not 16-byte aligned, no peer access, and the
  cross-check of the tests): the classic block scan over ranks:
      1. each rank reduces its slice to a carry per row, (P, S) = (product of the
         gates, last state from a zero start)                 -- `ascan_reduce_forward`
      2. ONE all_gather of the carries (plus the first gate of each slice, which the
         backward needs as its right halo): 3 values per row per rank
      3. each rank folds the carries of the ranks before it into its incoming state
         (`ascan_fold_carries`) and runs the scan seeded with it -- `ascan_forward(carry_in)`
  The backward mirrors it with the ranks after it: `ascan_reduce_backward`, one
  all_gather of (P', S'), a suffix fold, and the seeded fused backward
  (`carry_in`, `halo_gate_right`, `halo_state_left`).

The fold helpers are plain tensor arithmetic and run on any device; the local steps
default to the CUDA kernels (`NativeOps`) and fail on CPU tensors.  Tests inject other
local steps to exercise the exchange logic on CPU ranks (gloo).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import _native


def describe_exchange(single_pass: bool = True) -> str:
    """One line for benchmark records: what crosses the GPUs per step."""
    if single_pass:
        return ("peer stores of tagged 64-bit words: slice aggregate (P, S) per row to every later rank, forward "
                "and backward, plus the first gate of every row to the rank before (backward); no collective")
    return "all_gather of 3 (forward) + 2 (backward) fp32 per row per rank"


class PeerExchange:
    """Exchange buffers of the single-pass time-sharded scan for one process group, one row
    count and one device: a forward and a backward buffer per rank, allocated as peer-visible
    device memory, their inter-process handles exchanged once over the group (host side), and
    every rank's buffers mapped into every process.  Calls are numbered per direction; all
    ranks make the same calls in the same order, as with any collective."""

    _cache = {}

    def __init__(self, group, rows: int, device: torch.device):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.rows = rows
        self.device = device
        self.nbytes = (_native.exchange_bytes(rows, self.world) + 255) // 256 * 256
        self.calls = [0, 0]
        self.local = None
        self.opened = []
        ok, handle = 1, b""
        try:
            with torch.cuda.device(device):
                self.local, handle = _native.peer_alloc(2 * self.nbytes)
        except RuntimeError:
            ok = 0
        handles = [None] * self.world
        dist.all_gather_object(handles, (ok, handle), group=group)
        ptrs = [None] * self.world
        if all(h[0] for h in handles):
            try:
                with torch.cuda.device(device):
                    for j, (_, h) in enumerate(handles):
                        if j == self.rank:
                            ptrs[j] = self.local
                        else:
                            ptrs[j] = _native.peer_open(h)
                            self.opened.append(ptrs[j])
            except RuntimeError:
                ok = 0
        else:
            ok = 0
        # every rank must take the same path: one more round on the host
        flags = [None] * self.world
        dist.all_gather_object(flags, ok, group=group)
        self.usable = all(flags)
        if self.usable:
            self.fwd = ptrs
            self.bwd = [p + self.nbytes for p in ptrs]
        else:
            self.close()        # (every rank gets here together: the flags were gathered)

    def unmap(self):
        """Unmaps the other ranks' buffers from this process."""
        for p in self.opened:
            try:
                _native.peer_close(p)
            except RuntimeError:
                pass
        self.opened = []
        self.usable = False

    def release(self):
        """Frees this rank's own buffer.  Call it after every rank has unmapped (a buffer must
        not be freed while another process still maps it)."""
        if self.local is not None:
            try:
                _native.peer_free(self.local)
            except RuntimeError:
                pass
            self.local = None
        self.usable = False

    def close(self):
        """unmap, a host barrier of the group, release: collective over the group."""
        self.unmap()
        if dist.is_initialized():
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        self.release()

    def next_call(self, backward: bool) -> int:
        self.calls[int(backward)] += 1
        return self.calls[int(backward)]

    @classmethod
    def get(cls, group, rows: int, device: torch.device):
        key = (id(group) if group is not None else None, rows, device.index)
        ex = cls._cache.get(key)
        if ex is None:
            ex = cls(group, rows, device)
            cls._cache[key] = ex
        return ex

    @classmethod
    def close_all(cls):
        """Closes every exchange of this process (collective: all ranks call it at the same point)."""
        for ex in cls._cache.values():
            ex.close()
        cls._cache.clear()


def single_pass_supported(gates: torch.Tensor) -> bool:
    """The single-pass kernels use bulk copies: slices must be 16-byte aligned row by row."""
    return (gates.is_cuda and gates.data_ptr() % 16 == 0 and (gates.shape[-1] * gates.element_size()) % 16 == 0
            and gates.shape[-1] >= 1)


def shard_rows(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The rows of a (B, C, T) tensor that `rank` owns when B*C rows are dealt in
    contiguous blocks: returns a (1, rows_local, T) view-copy-free slice."""
    B, C, T = t.shape
    rows = B * C
    lo = rows * rank // world
    hi = rows * (rank + 1) // world
    return t.reshape(1, rows, T)[:, lo:hi]


def shard_time(t: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """The time slice of a (B, C, T) tensor that `rank` owns (contiguous copy)."""
    T = t.shape[-1]
    lo = T * rank // world
    hi = T * (rank + 1) // world
    return t[..., lo:hi].contiguous()


def compute_dtype(dtype: torch.dtype) -> torch.dtype:
    """Carries travel in the arithmetic type of the kernels."""
    return torch.complex64 if dtype == torch.complex64 else torch.float32


def fold_prefix(prod: torch.Tensor, state: torch.Tensor, rank: int) -> torch.Tensor:
    """Incoming state of `rank`: the composition of the carries of ranks 0..rank-1.
    prod, state: (world, rows).  x -> P*x + S applied in rank order from zero."""
    x = torch.zeros_like(state[0])
    for j in range(rank):
        x = prod[j] * x + state[j]
    return x


def fold_suffix(prod: torch.Tensor, state: torch.Tensor, rank: int) -> torch.Tensor:
    """Incoming adjoint of `rank` (g just after its last step): the composition of the
    backward carries of ranks world-1 down to rank+1."""
    world = prod.shape[0]
    g = torch.zeros_like(state[0])
    for j in range(world - 1, rank, -1):
        g = prod[j] * g + state[j]
    return g


class NativeOps:
    """The local steps on the CUDA kernels (C ABI)."""

    @staticmethod
    def reduce_forward(gates, tokens, payload):
        """Writes (P, S) of every row into payload[:, 0:2] (payload: (rows, >=2), compute dtype)."""
        rows = gates.numel() // gates.shape[-1]
        carry = torch.empty(rows, 2, dtype=payload.dtype, device=gates.device)
        _native.reduce_forward(gates, tokens, carry)
        payload[:, 0:2] = carry

    @staticmethod
    def forward(gates, tokens, carry_in):
        out = torch.empty_like(tokens)
        _native.forward(gates, tokens, out, carry_in=carry_in)
        return out

    @staticmethod
    def reduce_backward(gates, grad_out, halo_gate_right, payload):
        rows = gates.numel() // gates.shape[-1]
        carry = torch.empty(rows, 2, dtype=payload.dtype, device=gates.device)
        _native.reduce_backward(gates, grad_out, halo_gate_right, carry)
        payload[:, 0:2] = carry

    @staticmethod
    def backward(gates, states, grad_out, carry_in, halo_gate_right, halo_state_left):
        d_gates = torch.empty_like(gates)
        d_tokens = torch.empty_like(gates)
        _native.backward(gates, states, grad_out, d_gates, d_tokens, carry_in=carry_in,
                         halo_gate_right=halo_gate_right, halo_state_left=halo_state_left)
        return d_gates, d_tokens

    @staticmethod
    def fold(gathered, rank, suffix, want_halo):
        """One small kernel instead of a chain of tensor ops (ascan_fold_carries)."""
        return _native.fold_carries(gathered, rank, suffix, want_halo)


def fold_with_tensor_ops(gathered, rank, suffix, want_halo):
    """The same fold with plain tensor arithmetic (any device); gathered: (world, rows, stride)."""
    prod, state = gathered[:, :, 0], gathered[:, :, 1]
    x = fold_suffix(prod, state, rank) if suffix else fold_prefix(prod, state, rank)
    halo = None
    if want_halo:
        world = gathered.shape[0]
        halo = gathered[rank + 1, :, 2].clone() if rank + 1 < world else torch.ones_like(x)
    return x.contiguous(), halo


def _all_gather(x: torch.Tensor, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    x = x.contiguous()
    out = torch.empty((world * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)       # concatenated along dim 0 (gloo and nccl)
    return out.view((world,) + tuple(x.shape))


def time_sharded_forward(gates, tokens, group=None, ops=NativeOps):
    """Forward of the time-sharded scan on this rank's slice.  Returns
    (states, carry_in, halo_gate_right); the last two are what the backward needs."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    cdt = compute_dtype(gates.dtype)
    rows = gates.numel() // gates.shape[-1]
    if world == 1:
        return ops.forward(gates, tokens, None), None, None
    payload = torch.empty(rows, 3, dtype=cdt, device=gates.device)          # (P, S, first gate) per row
    ops.reduce_forward(gates, tokens, payload)
    payload[:, 2] = gates.reshape(rows, -1)[:, 0]
    gathered = _all_gather(payload, group)                                   # (world, rows, 3)
    carry_in, halo_gate_right = ops.fold(gathered, rank, False, True)
    states = ops.forward(gates, tokens, carry_in if rank > 0 else None)
    return states, carry_in, halo_gate_right


def time_sharded_backward(gates, states, grad_out, carry_in, halo_gate_right, group=None, ops=NativeOps):
    """Backward of the time-sharded scan on this rank's slice: (d_gates, d_tokens)."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world == 1:
        return ops.backward(gates, states, grad_out, None, None, None)
    cdt = compute_dtype(gates.dtype)
    rows = gates.numel() // gates.shape[-1]
    payload = torch.empty(rows, 2, dtype=cdt, device=gates.device)          # (P', S') per row
    ops.reduce_backward(gates, grad_out, halo_gate_right, payload)
    gathered = _all_gather(payload, group)                                   # (world, rows, 2)
    g_in, _ = ops.fold(gathered, rank, True, False)
    return ops.backward(gates, states, grad_out, g_in, halo_gate_right, carry_in)


def single_pass_forward(gates, tokens, exchange: PeerExchange):
    """This rank's slice, streamed once.  Returns (states, carry_in): carry_in is the state
    entering the slice, which the backward needs."""
    rows = gates.numel() // gates.shape[-1]
    states = torch.empty_like(tokens)
    carry_in = torch.empty(rows, dtype=compute_dtype(gates.dtype), device=gates.device)
    _native.forward_time_sharded(gates, tokens, states, exchange.rank, exchange.world, exchange.next_call(False),
                                 exchange.fwd, carry_in)
    return states, carry_in


def single_pass_backward(gates, states, grad_out, carry_in, exchange: PeerExchange):
    d_gates = torch.empty_like(gates)
    d_tokens = torch.empty_like(gates)
    _native.backward_time_sharded(gates, states, grad_out, d_gates, d_tokens, exchange.rank, exchange.world,
                                  exchange.next_call(True), exchange.bwd, carry_in)
    return d_gates, d_tokens


def _choose_single_pass(gates, tokens, group) -> PeerExchange | None:
    """The exchange buffers when every rank can take the single-pass path, else None.  The
    decision is made once per (group, row count, device) with one host-side round; after that
    it costs a dictionary look-up."""
    if not (single_pass_supported(gates) and single_pass_supported(tokens)):
        return None
    rows = gates.numel() // gates.shape[-1]
    ex = PeerExchange.get(group, rows, gates.device)
    return ex if ex.usable else None


class TimeShardedScan(torch.autograd.Function):
    """Autograd wrapper of the time-sharded scan (same contract as warp.Scan /
    complex.Scan on the local slice; `group` is the process group of the ranks that
    hold the slices of one sequence, in time order).  Every rank must hold a slice of the
    same length."""

    @staticmethod
    def forward(ctx, gates, tokens, group, single_pass=True):
        B, C, T = gates.shape
        assert tokens.shape == (B, C, T)
        assert gates.is_contiguous()
        assert tokens.is_contiguous()
        if gates.dtype != tokens.dtype:
            raise RuntimeError("gates and tokens must have the same dtype")
        ctx.group = group
        ctx.exchange = _choose_single_pass(gates, tokens, group) if (single_pass and dist.get_world_size(group) > 1) else None
        if ctx.exchange is not None:
            states, carry_in = single_pass_forward(gates, tokens, ctx.exchange)
            ctx.save_for_backward(gates, states, carry_in)
            return states
        states, carry_in, halo_gate_right = time_sharded_forward(gates, tokens, group)
        ctx.save_for_backward(gates, states, carry_in, halo_gate_right)
        return states

    @staticmethod
    def backward(ctx, grad_output):
        grad_output = grad_output.contiguous()
        if ctx.exchange is not None:
            gates, states, carry_in = ctx.saved_tensors
            d_gates, d_tokens = single_pass_backward(gates, states, grad_output, carry_in, ctx.exchange)
            return d_gates, d_tokens, None, None
        gates, states, carry_in, halo_gate_right = ctx.saved_tensors
        d_gates, d_tokens = time_sharded_backward(gates, states, grad_output, carry_in, halo_gate_right, ctx.group)
        return d_gates, d_tokens, None, None


def sharded_scan(gates, tokens, group=None, dim: str = "time", single_pass: bool = True):
    """Scan over tensors that are sharded across the ranks of `group`.

    dim="rows": the local tensors hold different rows; this is the plain single-GPU scan.
    dim="time": the local tensors hold consecutive time slices of equal length of the same
                rows (rank order = time order).  single_pass=True streams every slice once and
                exchanges slice aggregates by peer stores; False (and every case the single
                pass cannot take) runs the three-step scheme with one all_gather per direction.
    """
    if dim == "rows":
        if gates.dtype == torch.complex64:
            from . import complex as _complex
            return _complex.scan(gates, tokens)
        from . import warp as _warp
        return _warp.scan(gates, tokens)
    if dim != "time":
        raise ValueError("dim must be 'rows' or 'time'")
    return TimeShardedScan.apply(gates, tokens, group, single_pass)
