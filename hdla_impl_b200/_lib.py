"""ctypes binding of libhdla.so (C ABI declared in include/hdla.h).

There is no fallback: if the library is missing it is built with nvcc once; if that is not
possible, or a call fails, a ``RuntimeError`` carrying ``hdla_last_error()`` is raised.
"""
from __future__ import annotations

import ctypes as C
import os
import threading
from typing import Optional

import torch

HDLA_F32, HDLA_BF16 = 0, 1
FLAG_WS_HOLDS_FWD = 1
FLAG_FORCE_SIMT = 2
FLAG_FUSED_PREP = 4
FLAG_PARAM_AB = 8
FLAG_NORM_K = 256
PHASE_ALL, PHASE_PRE, PHASE_TRANSITION, PHASE_STATE, PHASE_POST = 0x00, 0x10, 0x20, 0x30, 0x40

EXPORTS = (
    "hdla_version", "hdla_last_error", "hdla_chunk_workspace_bytes", "hdla_chunk_fwd", "hdla_chunk_bwd",
    "hdla_recurrent_fwd", "hdla_chunk_uses_tensor_cores", "hdla_chunk_fwd_noalloc", "hdla_noalloc_read_status",
    "hdla_recurrent_read_status", "hdla_compose_states", "hdla_param_ab_fwd", "hdla_param_ab_bwd",
    "hdla_norm_gate_fwd", "hdla_norm_gate_bwd",
    # include/hdla_debug.h
    "hdla_kernel_launches", "hdla_timing_enable", "hdla_timing_report", "hdla_debug_tc_buffer",
    "hdla_debug_wait_timeout",
)


class HdlaDims(C.Structure):
    """Mirror of the C struct (include/hdla.h).  ``cu_seqlens`` points to HOST memory; ``with_seqlens`` keeps the
    array it points to alive for as long as the structure lives."""
    _fields_ = ([(n, C.c_int32) for n in ("B", "T", "H", "K", "V", "R", "C", "dtype", "gk_dtype", "flags",
                                          "n_seqs", "reserved_")]
                + [("cu_seqlens", C.POINTER(C.c_int64))])

    def with_seqlens(self, offsets) -> "HdlaDims":
        arr = (C.c_int64 * len(offsets))(*[int(x) for x in offsets])
        self._keep = arr
        self.n_seqs = len(offsets) - 1
        self.cu_seqlens = C.cast(arr, C.POINTER(C.c_int64))
        return self


_lock = threading.Lock()
_lib: Optional[C.CDLL] = None


def lib_path() -> str:
    return os.environ.get("HDLA_LIB") or os.path.join(os.path.dirname(os.path.abspath(__file__)), "libhdla.so")


def load() -> C.CDLL:
    """Load (building first if needed) the shared library and declare its prototypes."""
    global _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not os.path.exists(path):
            if os.environ.get("HDLA_LIB"):
                raise RuntimeError(f"HDLA_LIB={path} does not exist")
            from . import build as _build
            _build.build()
        lib = C.CDLL(path)
        vp, f32p = C.c_void_p, C.c_void_p
        dp = C.POINTER(HdlaDims)
        lib.hdla_version.restype = C.c_int
        lib.hdla_version.argtypes = []
        lib.hdla_last_error.restype = C.c_char_p
        lib.hdla_last_error.argtypes = []
        lib.hdla_kernel_launches.restype = C.c_ulonglong
        lib.hdla_kernel_launches.argtypes = []
        lib.hdla_param_ab_fwd.restype = C.c_int
        lib.hdla_param_ab_fwd.argtypes = [vp, vp, vp, vp, vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, vp]
        lib.hdla_param_ab_bwd.restype = C.c_int
        lib.hdla_param_ab_bwd.argtypes = [vp] * 8 + [C.c_int32] * 5 + [vp]
        lib.hdla_norm_gate_fwd.restype = C.c_int
        lib.hdla_norm_gate_fwd.argtypes = [vp, vp, vp, vp, C.c_int64, C.c_int32, C.c_float, C.c_int32, vp]
        lib.hdla_norm_gate_bwd.restype = C.c_int
        lib.hdla_norm_gate_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, C.c_int64, C.c_int32, C.c_float, C.c_int32, vp]
        lib.hdla_timing_enable.restype = None
        lib.hdla_timing_enable.argtypes = [C.c_int]
        lib.hdla_timing_report.restype = C.c_size_t
        lib.hdla_timing_report.argtypes = [C.c_char_p, C.c_size_t]
        lib.hdla_chunk_uses_tensor_cores.restype = C.c_int
        lib.hdla_chunk_uses_tensor_cores.argtypes = [dp]
        lib.hdla_debug_tc_buffer.restype = C.c_int
        lib.hdla_debug_tc_buffer.argtypes = [dp, vp, C.c_char_p, vp, vp]
        lib.hdla_chunk_workspace_bytes.restype = C.c_size_t
        lib.hdla_chunk_workspace_bytes.argtypes = [dp, C.c_int]
        lib.hdla_chunk_fwd.restype = C.c_int
        lib.hdla_chunk_fwd.argtypes = [dp, vp, vp, vp, vp, vp, vp, C.c_float, f32p, vp, f32p, vp, C.c_size_t, vp]
        lib.hdla_chunk_fwd_noalloc.restype = C.c_int
        lib.hdla_chunk_fwd_noalloc.argtypes = [dp, vp, vp, vp, vp, vp, vp, C.c_float, f32p, vp, f32p, vp]
        lib.hdla_noalloc_read_status.restype = C.c_int
        lib.hdla_noalloc_read_status.argtypes = [vp, vp]
        lib.hdla_recurrent_read_status.restype = C.c_int
        lib.hdla_recurrent_read_status.argtypes = [vp, vp]
        lib.hdla_compose_states.restype = C.c_int
        lib.hdla_compose_states.argtypes = [dp, vp, vp, vp, vp, vp, vp, C.c_int32, C.c_int64, C.c_int64, C.c_int32, vp]
        lib.hdla_debug_wait_timeout.restype = C.c_int
        lib.hdla_debug_wait_timeout.argtypes = [vp, C.c_uint64, vp]
        lib.hdla_chunk_bwd.restype = C.c_int
        lib.hdla_chunk_bwd.argtypes = [dp, vp, vp, vp, vp, vp, vp, C.c_float, f32p, vp, f32p,
                                       vp, vp, vp, vp, vp, vp, f32p, vp, C.c_size_t, vp]
        lib.hdla_recurrent_fwd.restype = C.c_int
        lib.hdla_recurrent_fwd.argtypes = [dp, vp, vp, vp, vp, vp, vp, C.c_float, f32p, vp, f32p,
                                           vp, C.c_int32, C.c_int32, vp]
        _lib = lib
        return lib


def kernel_launches() -> int:
    return int(load().hdla_kernel_launches())


def timing_enable(on: bool) -> None:
    load().hdla_timing_enable(int(on))


def timing_report() -> dict:
    """{kernel name: (launches, total ms)} since timing was enabled; waits for the recorded events."""
    buf = C.create_string_buffer(1 << 16)
    load().hdla_timing_report(buf, len(buf))
    out = {}
    for line in buf.value.decode().splitlines():
        name, cnt, ms = line.rsplit(" ", 2)
        out[name] = (int(cnt), float(ms))
    return out


def last_error() -> str:
    return load().hdla_last_error().decode("utf-8", "replace")


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed (code {rc}): {last_error()}")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float32:
        return HDLA_F32
    if dt == torch.bfloat16:
        return HDLA_BF16
    raise TypeError(f"libhdla supports float32 and bfloat16 tensors, got {dt}")


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(device) -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors) -> torch.device:
    dev = None
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("hdla_impl_b200 runs on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise RuntimeError(f"tensors on different devices: {dev} and {t.device}")
    return dev
