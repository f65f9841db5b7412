"""Chunked HDLA operator: ``chunk_hrdplr_delta_rule`` and its autograd function.

Same names, argument order, defaults and return values as the reference's
``HRDPLR/hrdplr.py:286-318`` (entry point) and ``:101-284`` (``ChunkDPLRDeltaRuleFunction``); the
stage sequence itself runs inside libhdla (``hdla_chunk_fwd`` / ``hdla_chunk_bwd``).
"""
from __future__ import annotations

import ctypes as C
import functools
import os
import warnings
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


def _tc_shape(q, v, RANK_AB: int) -> bool:
    """Whether the bf16 tensor-core pipeline takes this problem (at its own chunk of 64): bf16, rank 2, head dims
    that are multiples of 8 up to 128 (smaller ones run zero-padded on the same 128-wide tiles)."""
    T, K, V = q.shape[1], q.shape[-1], v.shape[-1]
    return (q.dtype == torch.bfloat16 and RANK_AB == 2 and K % 8 == 0 and V % 8 == 0 and 8 <= K <= 128
            and 8 <= V <= 128 and T > 32)


def _internal_chunk(q, v, RANK_AB: int, chunk_size: int) -> int:
    """Chunk size actually used.  The operator's result does not depend on the chunk size (it only sets how
    the recurrence is blocked), and the reference layer asks for 16 (HRDPLR/hdla_custom.py:308) only because its
    own backward is limited to that.  Problems the tensor-core pipeline supports are therefore run at its chunk
    of 64 whatever was requested; ``HDLA_HONOR_CHUNK=1`` keeps the requested value."""
    if (os.environ.get("HDLA_HONOR_CHUNK", "0") != "1" and _tc_shape(q, v, RANK_AB)
            and os.environ.get("HDLA_FORCE_SIMT", "0") != "1"):
        return 64
    return chunk_size


def _dims(q, v, a, gk, RANK_AB: int, chunk_size: int, flags: int = 0, cu_seqlens=None) -> _lib.HdlaDims:
    chunk_size = _internal_chunk(q, v, RANK_AB, chunk_size)
    B, T, H, K = q.shape
    if os.environ.get("HDLA_FORCE_SIMT", "0") == "1":      # debugging aid: fp32 CUDA-core pipeline for any dtype
        flags |= _lib.FLAG_FORCE_SIMT
    if os.environ.get("HDLA_FUSED_PREP", "0") == "1":      # one-kernel chunk preparation (see include/hdla.h)
        flags |= _lib.FLAG_FUSED_PREP
    d = _lib.HdlaDims(B, T, H, K, v.shape[-1], RANK_AB, chunk_size, _lib.dtype_code(q.dtype),
                      _lib.dtype_code(gk.dtype), flags)
    if cu_seqlens is not None:
        d.with_seqlens(cu_seqlens)
    return d


def _seq_offsets(cu_seqlens):
    """cu_seqlens (tensor or sequence of ints) -> tuple of python ints, or None.  The library sizes its grids from
    the offsets, so they are needed on the host (a device tensor is copied, which synchronises -- as the
    reference's chunk-index preparation does)."""
    if cu_seqlens is None:
        return None
    if isinstance(cu_seqlens, torch.Tensor):
        cu_seqlens = cu_seqlens.detach().cpu().tolist()
    return tuple(int(x) for x in cu_seqlens)


def _check_shapes(q, k, v, a, b, gk, RANK_AB, initial_state, n_states=None):
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
    N = B if n_states is None else n_states
    if initial_state is not None and initial_state.shape != (N, H, K, v.shape[-1]):
        raise ValueError(f"initial_state {tuple(initial_state.shape)} must be [{N}, H, K, V] = "
                         f"{(N, H, K, v.shape[-1])}")


def workspace_bytes(dims: _lib.HdlaDims, with_backward: bool) -> int:
    n = _lib.load().hdla_chunk_workspace_bytes(C.byref(dims), int(with_backward))
    if n == 0:
        raise RuntimeError(f"unsupported problem: {_lib.last_error()}")
    return n


# ---- device status words ----------------------------------------------------------------------
# The bf16 tensor-core kernels report in the first bytes of the workspace (see include/hdla.h):
# word 0 a device-side wait that ran out, word 1 a chunk whose total log decay is beyond what the
# pipeline represents, word 2 the largest chunk decay of the call.  After every launch the words are
# copied to pinned host memory without blocking and inspected the next time this module is entered on
# that device, so a problem never stays silent and the hot path never waits.
#
# A decay overflow is different from the other conditions: the call's results are wrong but the fp32
# pipeline would have computed them correctly (the reference layer feeds undivided logsigmoid decays,
# HRDPLR/hdla_custom.py:219, which can exceed the limit for fast-forgetting channels).  Forward
# therefore WAITS for its own status words -- and reruns the call on the fp32 pipeline when word 1 is
# set -- whenever an overflow is plausible: on the first call on a device, and from then on while the
# largest chunk decay seen on that device is above half the limit.  Workloads far from the limit (all
# benchmark configurations: <= 22 of 150) pay for one synchronisation in their first call only.
# HDLA_STRICT=1 always waits; HDLA_ASYNC_STATUS=1 never does (an overflow then raises at the next entry).
_RING = 64
_DECAY_LIMIT = 150.0
_status = {}      # device index -> dict(host=pinned [RING,4] int32, events=[...], next=int, pending=[slots], decay=float|None)
_warned_fallback = False


def _status_state(dev):
    st = _status.get(dev.index)
    if st is None:
        st = dict(host=torch.zeros(_RING, 4, dtype=torch.int32).pin_memory(),
                  events=[torch.cuda.Event() for _ in range(_RING)], next=0, pending=[], decay=None)
        _status[dev.index] = st
    return st


def _note_decay(st, words) -> None:
    seen = float(torch.tensor(int(words[2]), dtype=torch.int32).view(torch.float32))
    if seen == seen:
        st["decay"] = seen if st["decay"] is None else max(st["decay"], seen)


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
                _note_decay(st, words)
                if words[0] or words[1]:
                    st["pending"] = [s_ for s_ in st["pending"] if s_ != slot]
                    _raise_status(words)
            else:
                keep.append(slot)
        st["pending"] = keep


def _post_status(ws: torch.Tensor, dev) -> int:
    """Enqueue the copy of the status words of the call that just used ``ws``; returns the ring slot."""
    st = _status_state(dev)
    slot = st["next"]
    st["next"] = (slot + 1) % _RING
    if slot in st["pending"]:                       # ring wrapped: that copy finished long ago
        st["events"][slot].synchronize()
        check_status(dev)
    st["host"][slot].copy_(ws[:16].view(torch.int32), non_blocking=True)
    st["events"][slot].record(torch.cuda.current_stream(dev))
    st["pending"].append(slot)
    if os.environ.get("HDLA_STRICT", "0") == "1" and not torch.cuda.is_current_stream_capturing():
        check_status(dev, wait=True)
    return slot


def _overflow_plausible(dev) -> bool:
    if os.environ.get("HDLA_ASYNC_STATUS", "0") == "1" or torch.cuda.is_current_stream_capturing():
        return False
    st = _status_state(dev)
    return st["decay"] is None or st["decay"] > 0.5 * _DECAY_LIMIT or os.environ.get("HDLA_STRICT", "0") == "1"


def _wait_words(dev, slot):
    """Wait for the status copy in ``slot`` and take it off the pending list; returns its words."""
    st = _status_state(dev)
    st["events"][slot].synchronize()
    words = st["host"][slot].tolist()
    st["pending"] = [s_ for s_ in st["pending"] if s_ != slot]
    _note_decay(st, words)
    return words


def _alloc_ws(nbytes: int, device) -> torch.Tensor:
    return torch.empty(nbytes, dtype=torch.uint8, device=device)


def save_workspace_default() -> bool:
    """Whether forward keeps its intermediates for backward (default) or backward recomputes them
    like the reference does (``HDLA_RECOMPUTE=1``; trades time for activation memory)."""
    return os.environ.get("HDLA_RECOMPUTE", "0") != "1"


def chunk_hrdplr_fwd(q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first, chunk_size):
    """Forward stage sequence (reference: HRDPLR/hrdplr.py:25-99). Returns ``(o, final_state)``."""
    o, ht, _, _ = _chunk_fwd(q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first,
                             chunk_size)
    return o, ht


def _chunk_fwd(q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first, chunk_size,
               _keep_ws: bool = False, _force_simt: bool = False, cu_seqlens=None):
    """``chunk_hrdplr_fwd`` returning ``(o, final_state, workspace, used_fp32_pipeline)``; with ``_keep_ws`` the
    workspace is sized for, and keeps what, ``hdla_chunk_bwd(HDLA_FLAG_WS_HOLDS_FWD)`` needs."""
    global _warned_fallback
    assert head_first is False, "head_first=True is not supported (as in the reference)"
    dev = _lib.require_cuda(q, k, v, a, b, gk, initial_state)
    N = None if cu_seqlens is None else len(cu_seqlens) - 1
    _check_shapes(q, k, v, a, b, gk, RANK_AB, initial_state, N)
    check_status(dev)
    lib = _lib.load()
    dims = _dims(q, v, a, gk, RANK_AB, chunk_size, _lib.FLAG_FORCE_SIMT if _force_simt else 0, cu_seqlens)
    B, T, H, K = q.shape
    V = v.shape[-1]
    h0 = None if initial_state is None else initial_state.to(torch.float32).contiguous()
    with torch.cuda.device(dev):
        ws = _alloc_ws(workspace_bytes(dims, _keep_ws), dev)
        o = torch.empty_like(v)
        ht = torch.empty(B if N is None else N, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
        rc = lib.hdla_chunk_fwd(C.byref(dims), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(a), _lib.ptr(b),
                                _lib.ptr(gk), float(scale), _lib.ptr(h0), _lib.ptr(o), _lib.ptr(ht),
                                _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
        _lib.check(rc, "hdla_chunk_fwd")
        if lib.hdla_chunk_uses_tensor_cores(C.byref(dims)):
            slot = _post_status(ws, dev)
            if _overflow_plausible(dev):
                words = _wait_words(dev, slot)
                if words[1] and not words[0]:
                    if not _warned_fallback:
                        _warned_fallback = True
                        warnings.warn("hdla_impl_b200: a chunk's total log decay exceeds what the bf16 tensor-core "
                                      "pipeline represents; such calls are rerun on the fp32 CUDA-core pipeline "
                                      "(correct, much slower)", RuntimeWarning, stacklevel=3)
                    del ws, o, ht
                    if cu_seqlens is not None:
                        _raise_status(words)           # the fp32 pipeline takes no packed batches: the caller's
                                                       # per-sequence path has to be used for such decays
                    return _chunk_fwd(q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB,
                                      head_first, chunk_size, _keep_ws=_keep_ws, _force_simt=True)
                if words[0] or words[1]:
                    _raise_status(words)
    return o, ht, (ws if _keep_ws else None), _force_simt


class ChunkDPLRDeltaRuleFunction(torch.autograd.Function):
    """Autograd wrapper (reference: HRDPLR/hrdplr.py:101-284): forward saves the inputs; backward
    receives ``(do, dht)`` and returns gradients for q,k,v,a,b,gk and the initial state."""

    @staticmethod
    @contiguous
    @autocast_custom_fwd
    def forward(ctx, q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first, chunk_size,
                cu_seqlens=None):
        keep = save_workspace_default() and any(
            isinstance(t, torch.Tensor) and t.requires_grad for t in (q, k, v, a, b, gk, initial_state))
        o, final_state, ctx.ws, ctx.force_simt = _chunk_fwd(q, k, v, a, b, gk, scale, initial_state, output_final_state,
                                                            RANK_AB, head_first, chunk_size, _keep_ws=keep,
                                                            cu_seqlens=cu_seqlens)
        ctx.cu_seqlens = cu_seqlens
        ctx.save_for_backward(q, k, v, a, b, gk, initial_state)
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
        if ctx.force_simt:                          # forward had to fall back to the fp32 pipeline: so does backward
            flags |= _lib.FLAG_FORCE_SIMT
        dims = _dims(q, v, a, gk, ctx.RANK_AB, ctx.chunk_size, flags, ctx.cu_seqlens)
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
            if lib.hdla_chunk_uses_tensor_cores(C.byref(dims)):
                _post_status(ws, dev)                # waits that ran out in the backward kernels surface too
        if dh0 is not None and initial_state.dtype != torch.float32:
            dh0 = dh0.to(initial_state.dtype)
        return dq, dk, dv, da, db, dgk, None, dh0, None, None, None, None, None


def _packed_supported(q, v, RANK_AB: int) -> bool:
    return _tc_shape(q, v, RANK_AB) and os.environ.get("HDLA_FORCE_SIMT", "0") != "1" \
        and os.environ.get("HDLA_HONOR_CHUNK", "0") != "1"


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
    cu_seqlens=None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Drop-in for the reference's ``chunk_hrdplr_delta_rule`` (HRDPLR/hrdplr.py:286-318).

    ``cu_seqlens`` (an extension; the reference plumbs it only into its chunk kernels, HRDPLR/fwd_triton.py:618-623,
    HRDPLR/bwd_triton.py:919-924): offsets of sequences packed along T in a batch of one, as in
    ``fused_recurrent_dplr_delta_rule``; ``initial_state`` / the final state are then ``[n_seqs, H, K, V]``.  bf16
    problems of the tensor-core pipeline run packed (chunks never straddle two sequences; one scan per sequence
    and head); anything else is computed sequence by sequence."""
    assert q.dtype == k.dtype == v.dtype
    scale = k.shape[-1] ** -0.5 if scale is None else scale
    offsets = _seq_offsets(cu_seqlens)
    if offsets is not None:
        if q.shape[0] != 1:
            raise ValueError(f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                             f"Please flatten variable-length inputs before processing.")
        if initial_state is not None and initial_state.shape[0] != len(offsets) - 1:
            raise ValueError(f"The number of initial states is expected to be equal to the number of input sequences, "
                             f"i.e., {len(offsets) - 1} rather than {initial_state.shape[0]}.")
        if offsets[0] != 0 or offsets[-1] != q.shape[1] or any(y < x for x, y in zip(offsets, offsets[1:])):
            raise ValueError(f"cu_seqlens {offsets} must rise from 0 to T={q.shape[1]}")
        if not _packed_supported(q, v, RANK_AB):
            outs, states = [], []
            for s_, (lo, hi) in enumerate(zip(offsets, offsets[1:])):
                if hi == lo:
                    states.append(initial_state[s_:s_ + 1].float() if initial_state is not None else
                                  q.new_zeros(1, q.shape[2], q.shape[3], v.shape[-1], dtype=torch.float32))
                    continue
                h0 = None if initial_state is None else initial_state[s_:s_ + 1]
                o_s, ht_s = ChunkDPLRDeltaRuleFunction.apply(
                    q[:, lo:hi], k[:, lo:hi], v[:, lo:hi], a[:, lo * RANK_AB:hi * RANK_AB],
                    b[:, lo * RANK_AB:hi * RANK_AB], gk[:, lo:hi], scale, h0, output_final_state, RANK_AB,
                    head_first, chunk_size)
                outs.append(o_s)
                states.append(ht_s)
            return torch.cat(outs, 1), (torch.cat(states, 0) if output_final_state else None)
    o, final_state = ChunkDPLRDeltaRuleFunction.apply(
        q, k, v, a, b, gk, scale, initial_state, output_final_state, RANK_AB, head_first, chunk_size, offsets)
    return o, final_state
