"""Host-side plumbing shared by the operator entry points: argument checks, workspace, status word."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_STATUS = {}
STATUS_NAMES = {1: "bad page-table entry", 2: "top-k / cache index out of range", 3: "device-side wait timed out",
                4: "internal inconsistency in a kernel launch"}


def require_cuda():
    if not torch.cuda.is_available():
        raise RuntimeError("pypto_b200 needs a CUDA device (sm_100a); there is no CPU fallback")


def check_tensor(t, name, dtype, shape=None, ndim=None):
    if not isinstance(t, torch.Tensor):
        raise ValueError(f"{name}: expected a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise RuntimeError(f"{name}: expected a CUDA tensor, got device {t.device}")
    if t.dtype != dtype:
        raise ValueError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError(f"{name}: tensor must be contiguous")
    if ndim is not None and t.dim() != ndim:
        raise ValueError(f"{name}: expected {ndim} dims, got shape {tuple(t.shape)}")
    if shape is not None:
        if t.dim() != len(shape) or any(s is not None and int(d) != int(s) for d, s in zip(t.shape, shape)):
            raise ValueError(f"{name}: expected shape {tuple(shape)}, got {tuple(t.shape)}")
    return t


def same_device(*tensors):
    dev = tensors[0].device
    for t in tensors:
        if t.device != dev:
            raise RuntimeError(f"all tensors must live on one device: {dev} vs {t.device}")
    return dev


def gemm_bf16(a: torch.Tensor, b: torch.Tensor, out_dtype=torch.float32) -> torch.Tensor:
    """bf16 [m, k] x bf16 [k, n] -> fp32 (or bf16) [m, n] on this library's tcgen05 kernel: the products of bf16
    numbers are exact in fp32 and the accumulation is fp32, so this is the fp32 product of the widened operands up to
    the order of the summation.  `b` may be a contiguous [k, n] matrix or the transposed view of a contiguous [n, k]
    one (a weight held one row per output column); k must be a multiple of 64, n of 8."""
    check_tensor(a, "gemm a", torch.bfloat16, ndim=2)
    if not isinstance(b, torch.Tensor) or b.dtype != torch.bfloat16 or b.dim() != 2 or b.shape[0] != a.shape[1]:
        raise ValueError(f"gemm b: expected a bf16 matrix with {a.shape[1]} rows, got {getattr(b, 'shape', None)}")
    if b.is_contiguous():
        layout = 0
    elif b.t().is_contiguous():
        layout = 1
    else:
        raise ValueError("gemm b: expected a contiguous matrix or the transposed view of one")
    if out_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError(f"gemm: out_dtype {out_dtype} is neither float32 nor bfloat16")
    m, k, n = int(a.shape[0]), int(a.shape[1]), int(b.shape[1])
    dev = same_device(a, b)
    out = torch.empty((m, n), dtype=out_dtype, device=dev)
    if m == 0:
        return out
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws_bytes = lib.dsv32_gemm_bf16_workspace_bytes(m, k, n)
        ws = workspace(max(int(ws_bytes), 256), dev)
        args = _lib.GemmBf16Args(ptr(a), ptr(b), ptr(out), ptr(ws), int(ws_bytes), ptr(status_word(dev)), m, k, n, layout,
                                 1 if out_dtype == torch.bfloat16 else 0)
        _lib.check(lib.dsv32_gemm_bf16(C.byref(args), stream_ptr(dev)), "gemm_bf16")
    return out


def gemm_bf16_fp32(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """bf16 x bf16 -> fp32 (see gemm_bf16)."""
    return gemm_bf16(a, b, torch.float32)


def gemm_i8(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """int8 [m, k] x int8 [k, n] -> int32 [m, n], exact, on this library's tcgen05 kernel (k a multiple of 128, n of 256)."""
    check_tensor(a, "gemm a", torch.int8, ndim=2)
    check_tensor(b, "gemm b", torch.int8, (a.shape[1], None))
    m, k, n = int(a.shape[0]), int(a.shape[1]), int(b.shape[1])
    dev = same_device(a, b)
    out = torch.empty((m, n), dtype=torch.int32, device=dev)
    if m == 0:
        return out
    lib = _lib.load()
    with torch.cuda.device(dev):
        args = _lib.GemmI8Args(ptr(a), ptr(b), ptr(out), ptr(status_word(dev)), m, k, n)
        _lib.check(lib.dsv32_gemm_i8(C.byref(args), stream_ptr(dev)), "gemm_i8")
    return out


_SIDE_STREAMS = {}


class side_stream:
    """Run an independent branch of an operator on a second stream of the device: `with fork:` makes the side
    stream wait for the work already enqueued on the current stream and makes it current inside the block; the
    caller then enqueues the other branch on the original stream and calls `fork.join()`, after which the original
    stream waits for the side branch (events only, so the pattern can be captured in a CUDA graph).  Tensors
    created inside the block belong to the side stream's allocator pool; keep them referenced until the join."""

    def __init__(self, device):
        key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
        if key not in _SIDE_STREAMS:
            _SIDE_STREAMS[key] = torch.cuda.Stream(device=key)
        self.side = _SIDE_STREAMS[key]
        self.main = None
        self.ctx = None

    def __enter__(self):
        self.main = torch.cuda.current_stream(self.side.device)
        self.side.wait_stream(self.main)
        self.ctx = torch.cuda.stream(self.side)
        self.ctx.__enter__()
        return self.side

    def __exit__(self, *exc):
        self.ctx.__exit__(*exc)
        if exc[0] is not None:   # the side branch failed half-way: the caller's stream still waits for what it enqueued
            self.join()
        return False

    def join(self):
        self.main.wait_stream(self.side)


def ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def stream_ptr(device):
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def workspace(nbytes, device):
    if nbytes <= 0:
        return None
    return torch.empty(int(nbytes), dtype=torch.uint8, device=device)


def status_word(device):
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    st = _STATUS.get(key)
    if st is None:
        st = torch.zeros(4, dtype=torch.int32, device=device)
        _STATUS[key] = st
    return st


def check_status(device=None, synchronize=True):
    """Raise RuntimeError if a kernel of this library recorded a device-side anomaly on `device`.
    Synchronises the device first (the status word is written by the kernels)."""
    require_cuda()
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if synchronize:
        torch.cuda.synchronize(device)
    st = status_word(device)
    vals = st.tolist()
    if vals[0] != 0:
        st.zero_()
        raise RuntimeError(f"dsv32 device status {vals[0]} ({STATUS_NAMES.get(vals[0], '?')}), detail {vals[1:3]}")


lib = _lib.load
check = _lib.check
