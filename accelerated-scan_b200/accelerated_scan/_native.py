"""ctypes binding of libascan_b200.so (C ABI in include/ascan_b200.h).

This is the only place the Python package touches native code.  It replaces the
reference's import-time JIT build (warp.py:13-28): the library is built ahead of
time by build.py and loaded here.  There is no fallback: if the library is
missing, importing this module raises.
"""
from __future__ import annotations

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
        ("team_size", ctypes.c_int32), ("reserved", ctypes.c_int32),
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
    return lib


lib = _load()

EXPORTS = (
    "ascan_version", "ascan_strerror", "ascan_forward", "ascan_backward", "ascan_reduce_forward",
    "ascan_reduce_backward", "ascan_workspace_bytes", "ascan_plan_describe", "ascan_check",
    "ascan_forward_no_alloc", "ascan_fold_carries", "ascan_forward_complex_real_tokens",
    "ascan_forward_sigmoid_gates", "ascan_backward_sigmoid_gates", "ascan_backward_complex_real_tokens",
)


def strerror(code: int) -> str:
    return lib.ascan_strerror(int(code)).decode()


def check(code: int, what: str) -> None:
    """Raise RuntimeError for a non-zero status, as TORCH_CHECK does in the
    reference (warp.cuh:396-401,409-421)."""
    if code != OK:
        raise RuntimeError(f"{what}: {strerror(code)} (ascan status {code})")


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODE[t.dtype]
    except KeyError:
        raise RuntimeError(f"unsupported dtype {t.dtype}: expected float32, bfloat16, float16 or complex64")


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(t: torch.Tensor):
    return ctypes.c_void_p(torch.cuda.current_stream(t.device).cuda_stream)


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("accelerated_scan runs on CUDA tensors only (no CPU path)")


_workspaces = {}


def workspace(device: torch.device, rows: int = 0, seqlen: int = 1, dtype: int = 0, kind: int = 0) -> torch.Tensor:
    """Scratch per (device, stream), owned by torch's allocator and zero-filled once
    when it is created (the kernels rearm it themselves).  It holds the status word,
    the work ticket and one carry record per row; launches on different streams get
    different workspaces because they may overlap."""
    nbytes = int(lib.ascan_workspace_bytes(int(rows), int(seqlen), int(dtype), int(kind)))
    stream = torch.cuda.current_stream(device).cuda_stream
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(4096, 2 * nbytes), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def plan(rows: int, seqlen: int, dtype: int, kind: int, aligned: bool = True, workspace: bool = True,
         sm_count: int = 148, reverse: bool = False, lookback: bool = True, team: bool = True) -> dict:
    pl = Plan()
    flags = (int(bool(aligned)) | (int(bool(workspace)) << 1) | (int(bool(reverse)) << 2) | (int(not lookback) << 3)
             | (int(not team) << 4))
    check(lib.ascan_plan_describe(rows, seqlen, dtype, kind, flags, sm_count, ctypes.byref(pl)),
          "ascan_plan_describe")
    return pl.as_dict()


def forward(gates, tokens, out, reverse=False, carry_in=None):
    _require_cuda(gates, tokens, out, carry_in)
    rows = gates.numel() // gates.shape[-1] if gates.shape[-1] else 0
    T = gates.shape[-1]
    with torch.cuda.device(gates.device):
        ws = workspace(gates.device, rows, T, dtype_code(gates), KIND_FORWARD)
        rc = lib.ascan_forward(_ptr(gates), _ptr(tokens), _ptr(out), rows, T, dtype_code(gates), int(bool(reverse)),
                               _ptr(carry_in), _ptr(ws), ws.numel(), _stream(gates))
    check(rc, "ascan_forward")


UNSUPPORTED = 2


def forward_complex_real_tokens(gates, tokens_real, out, reverse=False) -> bool:
    """complex64 gates, float32 tokens (imaginary part zero), complex64 out.  Returns False
    when the library has no fused kernel for this shape or alignment (the caller then promotes
    the tokens to complex and calls `forward`)."""
    _require_cuda(gates, tokens_real, out)
    rows = gates.numel() // gates.shape[-1] if gates.shape[-1] else 0
    T = gates.shape[-1]
    with torch.cuda.device(gates.device):
        ws = workspace(gates.device, rows, T, C64, KIND_FORWARD)
        rc = lib.ascan_forward_complex_real_tokens(_ptr(gates), _ptr(tokens_real), _ptr(out), rows, T,
                                                   int(bool(reverse)), _ptr(ws), ws.numel(), _stream(gates))
    if rc == UNSUPPORTED:
        return False
    check(rc, "ascan_forward_complex_real_tokens")
    return True


def backward_complex_real_tokens(gates, states, grad_out, d_gates, d_tokens_real) -> bool:
    """Fused complex backward that writes only the real part of the token gradient (float32).
    Returns False when the library has no fused kernel for this shape or alignment."""
    _require_cuda(gates, states, grad_out, d_gates, d_tokens_real)
    rows = gates.numel() // gates.shape[-1] if gates.shape[-1] else 0
    T = gates.shape[-1]
    with torch.cuda.device(gates.device):
        ws = workspace(gates.device, rows, T, C64, KIND_BACKWARD)
        rc = lib.ascan_backward_complex_real_tokens(_ptr(gates), _ptr(states), _ptr(grad_out), _ptr(d_gates),
                                                    _ptr(d_tokens_real), rows, T, _ptr(ws), ws.numel(), _stream(gates))
    if rc == UNSUPPORTED:
        return False
    check(rc, "ascan_backward_complex_real_tokens")
    return True


def forward_sigmoid_gates(gate_logits, tokens, out) -> bool:
    """out[t] = sigmoid(gate_logits[t]) * out[t-1] + tokens[t].  Returns False when the library
    has no fused kernel for this shape or alignment (the caller applies the sigmoid itself)."""
    _require_cuda(gate_logits, tokens, out)
    rows = gate_logits.numel() // gate_logits.shape[-1] if gate_logits.shape[-1] else 0
    T = gate_logits.shape[-1]
    with torch.cuda.device(gate_logits.device):
        ws = workspace(gate_logits.device, rows, T, dtype_code(gate_logits), KIND_FORWARD)
        rc = lib.ascan_forward_sigmoid_gates(_ptr(gate_logits), _ptr(tokens), _ptr(out), rows, T,
                                             dtype_code(gate_logits), _ptr(ws), ws.numel(), _stream(gate_logits))
    if rc == UNSUPPORTED:
        return False
    check(rc, "ascan_forward_sigmoid_gates")
    return True


def backward_sigmoid_gates(gate_logits, states, grad_out, d_logits, d_tokens) -> bool:
    """Fused backward of `forward_sigmoid_gates`: d_logits and d_tokens.  False when unsupported."""
    _require_cuda(gate_logits, states, grad_out, d_logits, d_tokens)
    rows = gate_logits.numel() // gate_logits.shape[-1] if gate_logits.shape[-1] else 0
    T = gate_logits.shape[-1]
    with torch.cuda.device(gate_logits.device):
        ws = workspace(gate_logits.device, rows, T, dtype_code(gate_logits), KIND_BACKWARD)
        rc = lib.ascan_backward_sigmoid_gates(_ptr(gate_logits), _ptr(states), _ptr(grad_out), _ptr(d_logits),
                                              _ptr(d_tokens), rows, T, dtype_code(gate_logits), _ptr(ws), ws.numel(),
                                              _stream(gate_logits))
    if rc == UNSUPPORTED:
        return False
    check(rc, "ascan_backward_sigmoid_gates")
    return True


def backward(gates, states, grad_out, d_gates, d_tokens, carry_in=None, halo_gate_right=None, halo_state_left=None):
    _require_cuda(gates, states, grad_out, d_gates, d_tokens, carry_in, halo_gate_right, halo_state_left)
    rows = gates.numel() // gates.shape[-1] if gates.shape[-1] else 0
    T = gates.shape[-1]
    with torch.cuda.device(gates.device):
        ws = workspace(gates.device, rows, T, dtype_code(gates), KIND_BACKWARD)
        rc = lib.ascan_backward(_ptr(gates), _ptr(states), _ptr(grad_out), _ptr(d_gates), _ptr(d_tokens), rows, T,
                                dtype_code(gates), _ptr(carry_in), _ptr(halo_gate_right), _ptr(halo_state_left),
                                _ptr(ws), ws.numel(), _stream(gates))
    check(rc, "ascan_backward")


def reduce_forward(gates, tokens, carry_out):
    _require_cuda(gates, tokens, carry_out)
    rows = gates.numel() // gates.shape[-1]
    with torch.cuda.device(gates.device):
        ws = workspace(gates.device, rows)
        rc = lib.ascan_reduce_forward(_ptr(gates), _ptr(tokens), _ptr(carry_out), rows, gates.shape[-1],
                                      dtype_code(gates), _ptr(ws), ws.numel(), _stream(gates))
    check(rc, "ascan_reduce_forward")


def reduce_backward(gates, grad_out, halo_gate_right, carry_out):
    _require_cuda(gates, grad_out, halo_gate_right, carry_out)
    rows = gates.numel() // gates.shape[-1]
    with torch.cuda.device(gates.device):
        ws = workspace(gates.device, rows)
        rc = lib.ascan_reduce_backward(_ptr(gates), _ptr(grad_out), _ptr(halo_gate_right), _ptr(carry_out), rows,
                                       gates.shape[-1], dtype_code(gates), _ptr(ws), ws.numel(), _stream(gates))
    check(rc, "ascan_reduce_backward")


def fold_carries(gathered, rank: int, suffix: bool, want_halo: bool = False):
    """gathered: (world, rows, stride) tensor of float32 or complex64 on the GPU.  Returns
    (state, halo_or_None), each of `rows` values."""
    _require_cuda(gathered)
    world, rows, stride = gathered.shape
    state = torch.empty(rows, dtype=gathered.dtype, device=gathered.device)
    halo = torch.empty(rows, dtype=gathered.dtype, device=gathered.device) if want_halo else None
    code = C64 if gathered.dtype == torch.complex64 else F32
    with torch.cuda.device(gathered.device):
        rc = lib.ascan_fold_carries(_ptr(gathered), rows, world, int(rank), stride, code, int(bool(suffix)),
                                    _ptr(state), _ptr(halo), _stream(gathered))
    check(rc, "ascan_fold_carries")
    return state, halo


def check_status(device=None) -> None:
    """Synchronise and raise if a bounded device-side wait expired in an earlier launch."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(device):
        ws = workspace(device)
        rc = lib.ascan_check(_ptr(ws), ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream))
    check(rc, "ascan_check")
