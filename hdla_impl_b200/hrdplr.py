"""Chunked HDLA operator: ``chunk_hrdplr_delta_rule`` and its autograd function.

Same names, argument order, defaults and return values as the reference's
``HRDPLR/hrdplr.py:286-318`` (entry point) and ``:101-284`` (``ChunkDPLRDeltaRuleFunction``); the
stage sequence itself runs inside libhdla (``hdla_chunk_fwd`` / ``hdla_chunk_bwd``).
"""
from __future__ import annotations

import ctypes as C
import functools
import os
from typing import Optional, Tuple

import torch

from . import _lib

autocast_custom_fwd = functools.partial(torch.amp.custom_fwd, device_type="cuda")
autocast_custom_bwd = functools.partial(torch.amp.custom_bwd, device_type="cuda")


def contiguous(fn):
    """Make every tensor argument contiguous (reference: HRDPLR/utils.py:14-25)."""
    @functools.wraps(fn)
    def wrapper(ctx, *args, **kwargs):
        return fn(ctx,
                  *(i if not isinstance(i, torch.Tensor) else i.contiguous() for i in args),
                  **{k: (v if not isinstance(v, torch.Tensor) else v.contiguous()) for k, v in kwargs.items()})
    return wrapper


def _internal_chunk(q, v, RANK_AB: int, chunk_size: int) -> int:
    """Chunk size actually used.  The operator's result does not depend on the chunk size (it only sets how
    the recurrence is blocked), and the reference layer asks for 16 (HRDPLR/hdla_custom.py:308) only because its
    own backward is limited to that.  Problems the tensor-core pipeline supports are therefore run at its chunk
    of 64 whatever was requested; ``HDLA_HONOR_CHUNK=1`` keeps the requested value."""
    T, K, V = q.shape[1], q.shape[-1], v.shape[-1]
    if (os.environ.get("HDLA_HONOR_CHUNK", "0") != "1" and q.dtype == torch.bfloat16 and RANK_AB == 2
            and K == 128 and V == 128 and T > 32 and os.environ.get("HDLA_FORCE_SIMT", "0") != "1"):
        return 64
    return chunk_size


def _dims(q, v, a, gk, RANK_AB: int, chunk_size: int, flags: int = 0) -> _lib.HdlaDims:
    chunk_size = _internal_chunk(q, v, RANK_AB, chunk_size)
    B, T, H, K = q.shape
    if os.environ.get("HDLA_FORCE_SIMT", "0") == "1":      # debugging aid: fp32 CUDA-core pipeline for any dtype
        flags |= _lib.FLAG_FORCE_SIMT
    return _lib.HdlaDims(B, T, H, K, v.shape[-1], RANK_AB, chunk_size, _lib.dtype_code(q.dtype),
                         _lib.dtype_code(gk.dtype), flags)


def _check_shapes(q, k, v, a, b, gk, RANK_AB, initial_state):
    B, T, H, K = q.shape
    if k.shape != q.shape or gk.shape != q.shape:
        raise ValueError(f"k {tuple(k.shape)} and gk {tuple(gk.shape)} must match q {tuple(q.shape)}")
    if v.shape[:3] != q.shape[:3]:
        raise ValueError(f"v {tuple(v.shape)} must be [B, T, H, V] with q {tuple(q.shape)}")
    if a.shape != (B, T * RANK_AB, H, K) or b.shape != a.shape:
        raise ValueError(f"a {tuple(a.shape)} / b {tuple(b.shape)} must be [B, T*RANK_AB, H, K] = "
                         f"{(B, T * RANK_AB, H, K)}")
    if not (a.dtype == b.dtype == q.dtype):
        raise TypeError("a and b must have the dtype of q, k, v")
    if initial_state is not None and initial_state.shape != (B, H, K, v.shape[-1]):
        raise ValueError(f"initial_state {tuple(initial_state.shape)} must be [B, H, K, V]")


def workspace_bytes(dims: _lib.HdlaDims, with_backward: bool) -> int:
    n = _lib.load().hdla_chunk_workspace_bytes(C.byref(dims), int(with_backward))
    if n == 0:
        raise RuntimeError(f"unsupported problem: {_lib.last_error()}")
    return n


# ---- device status words ----------------------------------------------------------------------
# The bf16 tensor-core kernels report two conditions in the first 8 bytes of the workspace (see
# include/hdla.h).  They are copied to pinned host memory right after the forward launch, without
# blocking, and inspected the next time this module is entered on that device (or at once with
# HDLA_STRICT=1, which synchronises): a problem never stays silent, and the hot path never waits.
_RING = 64
_status = {}      # device index -> dict(host=pinned [RING,2] int32, events=[...], next=int, pending=[slots])


def _status_state(dev):
    st = _status.get(dev.index)
    if st is None:
        st = dict(host=torch.zeros(_RING, 2, dtype=torch.int32).pin_memory(),
                  events=[torch.cuda.Event() for _ in range(_RING)], next=0, pending=[])
        _status[dev.index] = st
    return st


def _raise_status(words):
    if words[0]:
        raise RuntimeError(f"libhdla: a device-side wait ran out (code {int(words[0])}); the results of that call are invalid")
    if words[1]:
        raise RuntimeError(
            "libhdla: the total log decay of some chunk exceeds 150 in some channel, beyond what the bf16 "
            "tensor-core pipeline represents; the results of that call are invalid. Set HDLA_FORCE_SIMT=1 to "
            "use the fp32 pipeline, which has no such limit.")


def check_status(dev=None, wait: bool = False) -> None:
    """Raise if an earlier bf16 call on ``dev`` reported a problem. ``wait`` synchronises first."""
    devs = list(_status) if dev is None else [dev.index if isinstance(dev, torch.device) else int(dev)]
    for di in devs:
        st = _status.get(di)
        if st is None:
            continue
        keep = []
        for slot in st["pending"]:
            ev = st["events"][slot]
            if wait:
                ev.synchronize()
            if ev.query():
                words = st["host"][slot].tolist()
                if words[0] or words[1]:
                    st["pending"] = [s_ for s_ in st["pending"] if s_ != slot]
                    _raise_status(words)
            else:
                keep.append(slot)
        st["pending"] = keep


def _post_status(ws: torch.Tensor, dev) -> None:
    st = _status_state(dev)
    slot = st["next"]
    st["next"] = (slot + 1) % _RING
    if slot in st["pending"]:                       # ring wrapped: that copy finished long ago
        st["events"][slot].synchronize()
        check_status(dev)
    st["host"][slot].copy_(ws[:8].view(torch.int32), non_blocking=True)
    st["events"][slot].record(torch.cuda.current_stream(dev))
    st["pending"].append(slot)
    if os.environ.get("HDLA_STRICT", "0") == "1":
        check_status(dev, wait=True)


def _alloc_ws(nbytes: int, device) -> torch.Tensor:
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def save_workspace_default() -> bool:
    """Whether forward keeps its intermediates for backward (default) or backward recomputes them
    like the reference does (``HDLA_RECOMPUTE=1``; trades time for activation memory)."""
    return os.environ.get("HDLA_RECOMPUTE", "0") != "1"


def chunk_hrdplr_fwd(q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first,
                     chunk_size, _keep_ws: bool = False):
    """Forward stage sequence (reference: HRDPLR/hrdplr.py:25-99). Returns ``(o, final_state)``
    (and the workspace tensor when ``_keep_ws``)."""
    assert head_first is False, "head_first=True is not supported (as in the reference)"
    dev = _lib.require_cuda(q, k, v, a, b, gk, initial_state)
    _check_shapes(q, k, v, a, b, gk, RANK_AB, initial_state)
    check_status(dev)
    lib = _lib.load()
    dims = _dims(q, v, a, gk, RANK_AB, chunk_size)
    B, T, H, K = q.shape
    V = v.shape[-1]
    h0 = None if initial_state is None else initial_state.to(torch.float32).contiguous()
    with torch.cuda.device(dev):
        ws = _alloc_ws(workspace_bytes(dims, _keep_ws), dev)
        o = torch.empty_like(v)
        ht = torch.empty(B, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
        rc = lib.hdla_chunk_fwd(C.byref(dims), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(a), _lib.ptr(b),
                                _lib.ptr(gk), float(scale), _lib.ptr(h0), _lib.ptr(o), _lib.ptr(ht),
                                _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "hdla_chunk_fwd")
    if lib.hdla_chunk_uses_tensor_cores(C.byref(dims)):
        with torch.cuda.device(dev):
            _post_status(ws, dev)
    if _keep_ws:
        return o, ht, ws
    return o, ht


class ChunkDPLRDeltaRuleFunction(torch.autograd.Function):
    """Autograd wrapper (reference: HRDPLR/hrdplr.py:101-284): forward saves the inputs; backward
    receives ``(do, dht)`` and returns gradients for q,k,v,a,b,gk and the initial state."""

    @staticmethod
    @contiguous
    @autocast_custom_fwd
    def forward(ctx, q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first, chunk_size):
        keep = save_workspace_default() and any(
            isinstance(t, torch.Tensor) and t.requires_grad for t in (q, k, v, a, b, gk, initial_state))
        res = chunk_hrdplr_fwd(q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first,
                               chunk_size, _keep_ws=keep)
        o, final_state = res[0], res[1]
        ctx.save_for_backward(q, k, v, a, b, gk, initial_state)
        ctx.ws = res[2] if keep else None
        ctx.head_first = head_first
        ctx.scale = scale
        ctx.chunk_size = chunk_size
        ctx.output_final_state = output_final_state
        ctx.RANK_AB = RANK_AB
        return o.to(q.dtype), final_state

    @staticmethod
    @contiguous
    @autocast_custom_bwd
    def backward(ctx, do, dht):
        q, k, v, a, b, gk, initial_state = ctx.saved_tensors
        dev = q.device
        check_status(dev)
        lib = _lib.load()
        ws = ctx.ws
        ctx.ws = None
        flags = _lib.FLAG_WS_HOLDS_FWD if ws is not None else 0
        dims = _dims(q, v, a, gk, ctx.RANK_AB, ctx.chunk_size, flags)
        h0 = None if initial_state is None else initial_state.to(torch.float32).contiguous()
        if do.dtype != q.dtype:
            do = do.to(q.dtype)
        if dht is not None:
            dht = dht.to(torch.float32).contiguous()
        with torch.cuda.device(dev):
            if ws is None:
                ws = _alloc_ws(workspace_bytes(dims, True), dev)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            da, db, dgk = torch.empty_like(a), torch.empty_like(b), torch.empty_like(gk)
            dh0 = torch.empty_like(h0) if h0 is not None else None
            rc = lib.hdla_chunk_bwd(C.byref(dims), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(a), _lib.ptr(b),
                                    _lib.ptr(gk), float(ctx.scale), _lib.ptr(h0), _lib.ptr(do), _lib.ptr(dht),
                                    _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(da), _lib.ptr(db),
                                    _lib.ptr(dgk), _lib.ptr(dh0), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
        _lib.check(rc, "hdla_chunk_bwd")
        if dh0 is not None and initial_state.dtype != torch.float32:
            dh0 = dh0.to(initial_state.dtype)
        return dq, dk, dv, da, db, dgk, None, dh0, None, None, None, None


@torch.compiler.disable
def chunk_hrdplr_delta_rule(
    q: torch.Tensor,   # [B, T, H, K]
    k: torch.Tensor,   # [B, T, H, K]
    v: torch.Tensor,   # [B, T, H, V]
    a: torch.Tensor,   # [B, T * RANK_AB, H, K]
    b: torch.Tensor,   # [B, T * RANK_AB, H, K]
    gk: torch.Tensor,  # [B, T, H, K]  log decay
    RANK_AB: int,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,   # [B, H, K, V]
    output_final_state: bool = False,
    head_first: bool = False,
    chunk_size: int = 32,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Drop-in for the reference's ``chunk_hrdplr_delta_rule`` (HRDPLR/hrdplr.py:286-318)."""
    assert q.dtype == k.dtype == v.dtype
    scale = k.shape[-1] ** -0.5 if scale is None else scale
    o, final_state = ChunkDPLRDeltaRuleFunction.apply(
        q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first, chunk_size)
    return o, final_state
