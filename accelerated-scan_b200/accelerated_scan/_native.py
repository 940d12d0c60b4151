"""ctypes binding of libascan_b200.so (C ABI in include/ascan_b200.h).

This is the only place the Python package touches native code.  It replaces the
reference's import-time JIT build (warp.py:13-28): the library is built ahead of
time by build.py and loaded here.  There is no fallback: if the library is
missing, importing this module raises.
"""
from __future__ import annotations

import contextlib
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libascan_b200.so")

OK = 0
F32, BF16, F16, C64 = 0, 1, 2, 3
KIND_FORWARD, KIND_BACKWARD, KIND_REDUCE_FORWARD, KIND_REDUCE_BACKWARD = 0, 1, 2, 3

DTYPE_CODE = {
    torch.float32: F32,
    torch.bfloat16: BF16,
    torch.float16: F16,
    torch.complex64: C64,
}


class Plan(ctypes.Structure):
    _fields_ = [
        ("kernel", ctypes.c_int32), ("loader", ctypes.c_int32), ("chunks_per_lane", ctypes.c_int32),
        ("stages", ctypes.c_int32), ("warps_per_cta", ctypes.c_int32), ("grid", ctypes.c_int32),
        ("tile_elems", ctypes.c_int32), ("dynamic", ctypes.c_int32),
        ("team_size", ctypes.c_int32), ("row_grid", ctypes.c_int32),
        ("rows_per_item", ctypes.c_int64), ("row_groups", ctypes.c_int64), ("seg_elems", ctypes.c_int64),
        ("fine_elems", ctypes.c_int64), ("coarse_segs", ctypes.c_int64), ("fine_segs", ctypes.c_int64),
        ("segs_per_row", ctypes.c_int64), ("items", ctypes.c_int64),
        ("smem_bytes", ctypes.c_uint64), ("workspace_bytes", ctypes.c_uint64),
    ]

    def as_dict(self):
        return {name: getattr(self, name) for name, _ in self._fields_}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python accelerated-scan_b200/build.py` "
            "(nvcc, sm_100a).  There is no CPU or PyTorch fallback.")
    lib = ctypes.CDLL(LIB_PATH)
    vp, i64, i32, sz = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_size_t
    lib.ascan_version.restype = i32
    lib.ascan_strerror.restype = ctypes.c_char_p
    lib.ascan_strerror.argtypes = [i32]
    lib.ascan_forward.restype = i32
    lib.ascan_forward.argtypes = [vp, vp, vp, i64, i64, i32, i32, vp, vp, sz, vp]
    lib.ascan_backward.restype = i32
    lib.ascan_backward.argtypes = [vp, vp, vp, vp, vp, i64, i64, i32, vp, vp, vp, vp, sz, vp]
    lib.ascan_reduce_forward.restype = i32
    lib.ascan_reduce_forward.argtypes = [vp, vp, vp, i64, i64, i32, vp, sz, vp]
    lib.ascan_reduce_backward.restype = i32
    lib.ascan_reduce_backward.argtypes = [vp, vp, vp, vp, i64, i64, i32, vp, sz, vp]
    lib.ascan_workspace_bytes.restype = sz
    lib.ascan_workspace_bytes.argtypes = [i64, i64, i32, i32]
    lib.ascan_plan_describe.restype = i32
    lib.ascan_plan_describe.argtypes = [i64, i64, i32, i32, i32, i32, ctypes.POINTER(Plan)]
    lib.ascan_check.restype = i32
    lib.ascan_check.argtypes = [vp, vp]
    lib.ascan_forward_complex_real_tokens.restype = i32
    lib.ascan_forward_complex_real_tokens.argtypes = [vp, vp, vp, i64, i64, i32, vp, sz, vp]
    lib.ascan_fold_carries.restype = i32
    lib.ascan_fold_carries.argtypes = [vp, i64, i32, i32, i32, i32, i32, vp, vp, vp]
    lib.ascan_backward_complex_real_tokens.restype = i32
    lib.ascan_backward_complex_real_tokens.argtypes = [vp, vp, vp, vp, vp, i64, i64, vp, sz, vp]
    lib.ascan_forward_sigmoid_gates.restype = i32
    lib.ascan_forward_sigmoid_gates.argtypes = [vp, vp, vp, i64, i64, i32, vp, sz, vp]
    lib.ascan_backward_sigmoid_gates.restype = i32
    lib.ascan_backward_sigmoid_gates.argtypes = [vp, vp, vp, vp, vp, i64, i64, i32, vp, sz, vp]
    lib.ascan_forward_no_alloc.restype = i32
    lib.ascan_forward_no_alloc.argtypes = [vp, vp, vp, i64, i64, i32, i32, vp]
    lib.ascan_check_no_alloc.restype = i32
    lib.ascan_check_no_alloc.argtypes = [vp]
    u32 = ctypes.c_uint32
    lib.ascan_exchange_bytes.restype = sz
    lib.ascan_exchange_bytes.argtypes = [i64, i32]
    lib.ascan_workspace_bytes_time_sharded.restype = sz
    lib.ascan_workspace_bytes_time_sharded.argtypes = [i64, i64, i32, i32]
    lib.ascan_forward_time_sharded.restype = i32
    lib.ascan_forward_time_sharded.argtypes = [vp, vp, vp, i64, i64, i32, i32, i32, u32, vp, vp, vp, sz, vp]
    lib.ascan_backward_time_sharded.restype = i32
    lib.ascan_backward_time_sharded.argtypes = [vp, vp, vp, vp, vp, i64, i64, i32, i32, i32, u32, vp, vp, vp, sz, vp]
    lib.ascan_peer_alloc.restype = i32
    lib.ascan_peer_alloc.argtypes = [sz, ctypes.POINTER(ctypes.c_void_p), vp]
    lib.ascan_peer_open.restype = i32
    lib.ascan_peer_open.argtypes = [vp, ctypes.POINTER(ctypes.c_void_p)]
    lib.ascan_peer_close.restype = i32
    lib.ascan_peer_close.argtypes = [vp]
    lib.ascan_peer_free.restype = i32
    lib.ascan_peer_free.argtypes = [vp]
    lib.ascan_set_option.restype = i32
    lib.ascan_set_option.argtypes = [i32, i32]
    lib.ascan_get_option.restype = i32
    lib.ascan_get_option.argtypes = [i32]
    return lib


lib = _load()

EXPORTS = (
    "ascan_version", "ascan_strerror", "ascan_forward", "ascan_backward", "ascan_reduce_forward",
    "ascan_reduce_backward", "ascan_workspace_bytes", "ascan_plan_describe", "ascan_check",
    "ascan_forward_no_alloc", "ascan_fold_carries", "ascan_forward_complex_real_tokens",
    "ascan_forward_sigmoid_gates", "ascan_backward_sigmoid_gates", "ascan_backward_complex_real_tokens",
    "ascan_check_no_alloc", "ascan_set_option", "ascan_get_option",
    "ascan_exchange_bytes", "ascan_workspace_bytes_time_sharded", "ascan_forward_time_sharded",
    "ascan_backward_time_sharded", "ascan_peer_alloc", "ascan_peer_open", "ascan_peer_close", "ascan_peer_free",
)

(OPT_STAGES, OPT_WARPS_PER_CTA, OPT_LOOKBACK_TILES, OPT_DISABLE_PLANS, OPT_TEST_DROP_CARRY, OPT_TEST_EPOCH_BITS,
 OPT_ITEMS_PER_WARP, OPT_STATIC_BELOW) = range(8)


def strerror(code: int) -> str:
    return lib.ascan_strerror(int(code)).decode()


def check(code: int, what: str) -> None:
    """Raise RuntimeError for a non-zero status, as TORCH_CHECK does in the
    reference (warp.cuh:396-401,409-421)."""
    if code != OK:
        raise RuntimeError(f"{what}: {strerror(code)} (ascan status {code})")


def set_option(option: int, value: int) -> None:
    check(lib.ascan_set_option(int(option), int(value)), "ascan_set_option")


def get_option(option: int) -> int:
    return int(lib.ascan_get_option(int(option)))


# Debug mode: synchronise after every launch and raise if a bounded device-side wait
# expired in it (the reference raises on every failure, warp.cuh:396-421).  Off by
# default, because the hot path must not synchronise; without it a failure is still
# reported, one call late: see Workspace.raise_if_failed.
_debug = os.environ.get("ASCAN_CHECK", "") not in ("", "0")


def set_debug(on: bool) -> None:
    global _debug
    _debug = bool(on)


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {t.dtype}: expected float32, bfloat16, float16 or complex64")


def _ptr(t):
    return None if t is None else t.data_ptr()


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("accelerated_scan runs on CUDA tensors only (no CPU path)")


def _raw_stream(device) -> int:
    """cudaStream_t of torch's current stream on `device`, as an integer."""
    return torch._C._cuda_getCurrentRawStream(device.index)


def _rows_T(t):
    T = t.shape[-1]
    return (t.numel() // T if T else 0), T


_NULL_GUARD = contextlib.nullcontext()


def _device_guard(device):
    """The C ABI works on the current device: switch only when the tensors live elsewhere."""
    return _NULL_GUARD if torch.cuda.current_device() == device.index else torch.cuda.device(device)


class Workspace:
    """Scratch of one (device, stream), owned by torch's allocator and zero-filled once
    when it is created (the kernels rearm it themselves).  It holds the status word, the
    work ticket and the carry records; launches on different streams get different
    workspaces because they may overlap.  A word of pinned host memory is registered in
    the control block as second status word: a kernel whose bounded wait expires writes
    there too, so the failure is seen by a plain host read at the next call."""

    def __init__(self, device, nbytes):
        self.tensor = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        self.nbytes = nbytes
        self.ptr = self.tensor.data_ptr()
        self.sink = torch.zeros(4, dtype=torch.int32).pin_memory()
        self.sink_np = self.sink.numpy()
        self.tensor[16:24] = torch.tensor([self.sink.data_ptr()], dtype=torch.int64).view(torch.uint8).to(device)

    def raise_if_failed(self):
        if self.sink_np[0]:
            # reported here: clear both copies of the status (the device word in stream order)
            self.sink_np[0] = 0
            self.tensor[0:4].zero_()
            raise RuntimeError("accelerated_scan: a bounded device-side wait expired in an earlier launch on this "
                               "stream; its result is invalid (ascan status 4)")


_workspaces = {}
_needs = {}


def _workspace(device, stream, rows, seqlen, dtype, kind) -> Workspace:
    key = (rows, seqlen, dtype, kind)
    nbytes = _needs.get(key)
    if nbytes is None:
        nbytes = int(lib.ascan_workspace_bytes(rows, seqlen, dtype, kind))
        if len(_needs) > 4096:
            _needs.clear()
        _needs[key] = nbytes
    wkey = (device.index, stream)
    ws = _workspaces.get(wkey)
    if ws is None or ws.nbytes < nbytes:
        ws = Workspace(device, max(4096, 2 * nbytes))
        _workspaces[wkey] = ws
    ws.raise_if_failed()
    return ws


def workspace(device: torch.device, rows: int = 0, seqlen: int = 1, dtype: int = 0, kind: int = 0) -> torch.Tensor:
    """The scratch tensor launches on the current stream of `device` use (see Workspace)."""
    device = torch.device(device)
    stream = _raw_stream(device)
    return _workspace(device, stream, int(rows), int(seqlen), int(dtype), int(kind)).tensor


launch_count = 0       # kernels launched through this module (every successful call is one launch)


def _finish(rc, what, ws, stream):
    global launch_count
    check(rc, what)
    launch_count += 1
    if _debug:
        rc = lib.ascan_check(ws.ptr, stream)
        ws.sink_np[0] = 0
        check(rc, what)


def plan(rows: int, seqlen: int, dtype: int, kind: int, aligned: bool = True, workspace: bool = True,
         sm_count: int = 148, reverse: bool = False, lookback: bool = True, team: bool = True,
         seeded: bool = False) -> dict:
    pl = Plan()
    flags = (int(bool(aligned)) | (int(bool(workspace)) << 1) | (int(bool(reverse)) << 2) | (int(not lookback) << 3)
             | (int(not team) << 4) | (int(bool(seeded)) << 5))
    check(lib.ascan_plan_describe(rows, seqlen, dtype, kind, flags, sm_count, ctypes.byref(pl)),
          "ascan_plan_describe")
    return pl.as_dict()


def forward(gates, tokens, out, reverse=False, carry_in=None):
    _require_cuda(gates, tokens, out, carry_in)
    rows, T = _rows_T(gates)
    code = dtype_code(gates)
    dev = gates.device
    stream = _raw_stream(dev)
    ws = _workspace(dev, stream, rows, T, code, KIND_FORWARD)
    with _device_guard(dev):
        rc = lib.ascan_forward(gates.data_ptr(), tokens.data_ptr(), out.data_ptr(), rows, T, code, int(bool(reverse)),
                               _ptr(carry_in), ws.ptr, ws.nbytes, stream)
    _finish(rc, "ascan_forward", ws, stream)


UNSUPPORTED = 2


def forward_complex_real_tokens(gates, tokens_real, out, reverse=False) -> bool:
    """complex64 gates, float32 tokens (imaginary part zero), complex64 out.  Returns False
    when the library has no fused kernel for this shape or alignment (the caller then promotes
    the tokens to complex and calls `forward`)."""
    _require_cuda(gates, tokens_real, out)
    rows, T = _rows_T(gates)
    dev = gates.device
    stream = _raw_stream(dev)
    ws = _workspace(dev, stream, rows, T, C64, KIND_FORWARD)
    with _device_guard(dev):
        rc = lib.ascan_forward_complex_real_tokens(gates.data_ptr(), tokens_real.data_ptr(), out.data_ptr(), rows, T,
                                                   int(bool(reverse)), ws.ptr, ws.nbytes, stream)
    if rc == UNSUPPORTED:
        return False
    _finish(rc, "ascan_forward_complex_real_tokens", ws, stream)
    return True


def backward_complex_real_tokens(gates, states, grad_out, d_gates, d_tokens_real) -> bool:
    """Fused complex backward that writes only the real part of the token gradient (float32).
    Returns False when the library has no fused kernel for this shape or alignment."""
    _require_cuda(gates, states, grad_out, d_gates, d_tokens_real)
    rows, T = _rows_T(gates)
    dev = gates.device
    stream = _raw_stream(dev)
    ws = _workspace(dev, stream, rows, T, C64, KIND_BACKWARD)
    with _device_guard(dev):
        rc = lib.ascan_backward_complex_real_tokens(gates.data_ptr(), states.data_ptr(), grad_out.data_ptr(),
                                                    d_gates.data_ptr(), d_tokens_real.data_ptr(), rows, T, ws.ptr,
                                                    ws.nbytes, stream)
    if rc == UNSUPPORTED:
        return False
    _finish(rc, "ascan_backward_complex_real_tokens", ws, stream)
    return True


def forward_sigmoid_gates(gate_logits, tokens, out) -> bool:
    """out[t] = sigmoid(gate_logits[t]) * out[t-1] + tokens[t].  Returns False when the library
    has no fused kernel for this shape or alignment (the caller applies the sigmoid itself)."""
    _require_cuda(gate_logits, tokens, out)
    rows, T = _rows_T(gate_logits)
    code = dtype_code(gate_logits)
    dev = gate_logits.device
    stream = _raw_stream(dev)
    ws = _workspace(dev, stream, rows, T, code, KIND_FORWARD)
    with _device_guard(dev):
        rc = lib.ascan_forward_sigmoid_gates(gate_logits.data_ptr(), tokens.data_ptr(), out.data_ptr(), rows, T, code,
                                             ws.ptr, ws.nbytes, stream)
    if rc == UNSUPPORTED:
        return False
    _finish(rc, "ascan_forward_sigmoid_gates", ws, stream)
    return True


def backward_sigmoid_gates(gate_logits, states, grad_out, d_logits, d_tokens) -> bool:
    """Fused backward of `forward_sigmoid_gates`: d_logits and d_tokens.  False when unsupported."""
    _require_cuda(gate_logits, states, grad_out, d_logits, d_tokens)
    rows, T = _rows_T(gate_logits)
    code = dtype_code(gate_logits)
    dev = gate_logits.device
    stream = _raw_stream(dev)
    ws = _workspace(dev, stream, rows, T, code, KIND_BACKWARD)
    with _device_guard(dev):
        rc = lib.ascan_backward_sigmoid_gates(gate_logits.data_ptr(), states.data_ptr(), grad_out.data_ptr(),
                                              d_logits.data_ptr(), d_tokens.data_ptr(), rows, T, code, ws.ptr,
                                              ws.nbytes, stream)
    if rc == UNSUPPORTED:
        return False
    _finish(rc, "ascan_backward_sigmoid_gates", ws, stream)
    return True


def backward(gates, states, grad_out, d_gates, d_tokens, carry_in=None, halo_gate_right=None, halo_state_left=None):
    _require_cuda(gates, states, grad_out, d_gates, d_tokens, carry_in, halo_gate_right, halo_state_left)
    rows, T = _rows_T(gates)
    code = dtype_code(gates)
    dev = gates.device
    stream = _raw_stream(dev)
    ws = _workspace(dev, stream, rows, T, code, KIND_BACKWARD)
    with _device_guard(dev):
        rc = lib.ascan_backward(gates.data_ptr(), states.data_ptr(), grad_out.data_ptr(), d_gates.data_ptr(),
                                d_tokens.data_ptr(), rows, T, code, _ptr(carry_in), _ptr(halo_gate_right),
                                _ptr(halo_state_left), ws.ptr, ws.nbytes, stream)
    _finish(rc, "ascan_backward", ws, stream)


def reduce_forward(gates, tokens, carry_out):
    _require_cuda(gates, tokens, carry_out)
    rows, T = _rows_T(gates)
    code = dtype_code(gates)
    dev = gates.device
    stream = _raw_stream(dev)
    ws = _workspace(dev, stream, rows, T, code, KIND_REDUCE_FORWARD)
    with _device_guard(dev):
        rc = lib.ascan_reduce_forward(gates.data_ptr(), tokens.data_ptr(), carry_out.data_ptr(), rows, T, code,
                                      ws.ptr, ws.nbytes, stream)
    _finish(rc, "ascan_reduce_forward", ws, stream)


def reduce_backward(gates, grad_out, halo_gate_right, carry_out):
    _require_cuda(gates, grad_out, halo_gate_right, carry_out)
    rows, T = _rows_T(gates)
    code = dtype_code(gates)
    dev = gates.device
    stream = _raw_stream(dev)
    ws = _workspace(dev, stream, rows, T, code, KIND_REDUCE_BACKWARD)
    with _device_guard(dev):
        rc = lib.ascan_reduce_backward(gates.data_ptr(), grad_out.data_ptr(), _ptr(halo_gate_right),
                                       carry_out.data_ptr(), rows, T, code, ws.ptr, ws.nbytes, stream)
    _finish(rc, "ascan_reduce_backward", ws, stream)


def _sharded_workspace(dev, stream, rows, T, code, kind) -> Workspace:
    key = ("time_sharded", rows, T, code, kind)
    nbytes = _needs.get(key)
    if nbytes is None:
        nbytes = int(lib.ascan_workspace_bytes_time_sharded(rows, T, code, kind))
        _needs[key] = nbytes
    wkey = (dev.index, stream)
    ws = _workspaces.get(wkey)
    if ws is None or ws.nbytes < nbytes:
        ws = Workspace(dev, max(4096, 2 * nbytes))
        _workspaces[wkey] = ws
    ws.raise_if_failed()
    return ws


def forward_time_sharded(gates, tokens, out, rank: int, world: int, call: int, exchange_ptrs, carry_save=None):
    """This rank's slice of a time-sharded forward scan (ascan_forward_time_sharded).
    exchange_ptrs: `world` integers, the ranks' forward exchange buffers as mapped here."""
    _require_cuda(gates, tokens, out, carry_save)
    rows, T = _rows_T(gates)
    code = dtype_code(gates)
    dev = gates.device
    stream = _raw_stream(dev)
    ws = _sharded_workspace(dev, stream, rows, T, code, KIND_FORWARD)
    table = (ctypes.c_void_p * world)(*exchange_ptrs) if world > 1 else None
    with _device_guard(dev):
        rc = lib.ascan_forward_time_sharded(gates.data_ptr(), tokens.data_ptr(), out.data_ptr(), rows, T, code,
                                            int(rank), int(world), int(call), table, _ptr(carry_save), ws.ptr,
                                            ws.nbytes, stream)
    _finish(rc, "ascan_forward_time_sharded", ws, stream)


def backward_time_sharded(gates, states, grad_out, d_gates, d_tokens, rank: int, world: int, call: int, exchange_ptrs,
                          halo_state_left=None):
    """This rank's slice of the fused backward of a time-sharded scan (ascan_backward_time_sharded).
    exchange_ptrs: the ranks' backward exchange buffers; halo_state_left: carry_save of the forward."""
    _require_cuda(gates, states, grad_out, d_gates, d_tokens, halo_state_left)
    rows, T = _rows_T(gates)
    code = dtype_code(gates)
    dev = gates.device
    stream = _raw_stream(dev)
    ws = _sharded_workspace(dev, stream, rows, T, code, KIND_BACKWARD)
    table = (ctypes.c_void_p * world)(*exchange_ptrs) if world > 1 else None
    with _device_guard(dev):
        rc = lib.ascan_backward_time_sharded(gates.data_ptr(), states.data_ptr(), grad_out.data_ptr(), d_gates.data_ptr(),
                                             d_tokens.data_ptr(), rows, T, code, int(rank), int(world), int(call), table,
                                             _ptr(halo_state_left), ws.ptr, ws.nbytes, stream)
    _finish(rc, "ascan_backward_time_sharded", ws, stream)


def exchange_bytes(rows: int, world: int) -> int:
    return int(lib.ascan_exchange_bytes(int(rows), int(world)))


def peer_alloc(nbytes: int):
    """(device pointer, 64-byte inter-process handle) of a zero-filled peer-visible buffer."""
    ptr = ctypes.c_void_p()
    handle = ctypes.create_string_buffer(64)
    check(lib.ascan_peer_alloc(int(nbytes), ctypes.byref(ptr), handle), "ascan_peer_alloc")
    return int(ptr.value), handle.raw


def peer_open(handle: bytes) -> int:
    ptr = ctypes.c_void_p()
    check(lib.ascan_peer_open(ctypes.create_string_buffer(handle, 64), ctypes.byref(ptr)), "ascan_peer_open")
    return int(ptr.value)


def peer_close(ptr: int) -> None:
    check(lib.ascan_peer_close(ptr), "ascan_peer_close")


def peer_free(ptr: int) -> None:
    check(lib.ascan_peer_free(ptr), "ascan_peer_free")


def fold_carries(gathered, rank: int, suffix: bool, want_halo: bool = False):
    """gathered: (world, rows, stride) tensor of float32 or complex64 on the GPU.  Returns
    (state, halo_or_None), each of `rows` values."""
    _require_cuda(gathered)
    world, rows, stride = gathered.shape
    state = torch.empty(rows, dtype=gathered.dtype, device=gathered.device)
    halo = torch.empty(rows, dtype=gathered.dtype, device=gathered.device) if want_halo else None
    code = C64 if gathered.dtype == torch.complex64 else F32
    with _device_guard(gathered.device):
        rc = lib.ascan_fold_carries(gathered.data_ptr(), rows, world, int(rank), stride, code, int(bool(suffix)),
                                    state.data_ptr(), _ptr(halo), _raw_stream(gathered.device))
    check(rc, "ascan_fold_carries")
    return state, halo


def check_status(device=None) -> None:
    """Synchronise the current stream of `device` and raise if a bounded device-side wait
    expired in an earlier launch on it."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    stream = _raw_stream(device)
    ws = _workspaces.get((device.index, stream))
    if ws is None:
        return
    with _device_guard(device):
        rc = lib.ascan_check(ws.ptr, stream)
    ws.sink_np[0] = 0
    check(rc, "ascan_check")
