"""Fused recurrent HDLA forward: ``fused_recurrent_dplr_delta_rule`` (decode / short prefill).

Same signature, validation and return values as the reference's ``HRDPLR/recurrent.py:227-319``;
the recurrence runs in libhdla's ``hdla_recurrent_fwd``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from .hrdplr import autocast_custom_bwd, autocast_custom_fwd, contiguous


def fused_recurrent_dplr_delta_rule_fwd(q, k, v, a, b, gk, rank_ab, scale=1.0, initial_state=None,
                                        output_final_state=False, reverse=False, cu_seqlens=None,
                                        inplace_state: bool = False):
    """Reference: HRDPLR/recurrent.py:121-177. ``inplace_state`` writes the final state over
    ``initial_state`` (an fp32 tensor) instead of allocating a new one."""
    B, TR, H, K = a.shape
    T = _tokens_of_merged(TR, rank_ab)
    # same conditions and messages as the reference's wrapper (HRDPLR/recurrent.py:136-145)
    for name, t, want, text in (("b", b, (B, TR, H, K), f"doesn't match a shape {a.shape}"),
                                ("k", k, (B, T, H, K), "should be (B, T, H, K)"),
                                ("v", v, (B, T, H, v.shape[-1]), "should be (B, T, H, V)"),
                                ("q", q, (B, T, H, K), "should be (B, T, H, K)"),
                                ("gk", gk, (B, T, H, K), "should be (B, T, H, K)")):
        assert t.shape == want, f"{name} shape {t.shape} {text}"
    dev = _lib.require_cuda(q, k, v, a, b, gk, initial_state, cu_seqlens)
    if not (q.dtype == k.dtype == v.dtype == a.dtype == b.dtype):
        raise TypeError("q, k, v, a, b must share one dtype")
    V = v.shape[-1]
    N = B if cu_seqlens is None else len(cu_seqlens) - 1
    lib = _lib.load()
    dims = _lib.HdlaDims(B, T, H, K, V, rank_ab, 0, _lib.dtype_code(q.dtype), _lib.dtype_code(gk.dtype), 0)
    h0 = initial_state
    if h0 is not None:
        if inplace_state and (h0.dtype != torch.float32 or not h0.is_contiguous()):
            raise ValueError("inplace_state needs a contiguous float32 initial_state")
        h0 = h0.to(torch.float32).contiguous()
    cu = None if cu_seqlens is None else cu_seqlens.to(torch.int64).contiguous()
    with torch.cuda.device(dev):
        o = torch.empty_like(v)
        if inplace_state and h0 is not None:
            ht = h0
        else:
            ht = q.new_empty(N, H, K, V, dtype=torch.float32) if output_final_state else None
        rc = lib.hdla_recurrent_fwd(C.byref(dims), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(a), _lib.ptr(b),
                                    _lib.ptr(gk), float(scale), _lib.ptr(h0), _lib.ptr(o), _lib.ptr(ht),
                                    _lib.ptr(cu), N, int(bool(reverse)), _lib.stream_ptr(dev))
        _lib.check(rc, "hdla_recurrent_fwd")
        _poll_status(lib, dev)
    return o, ht


def _tokens_of_merged(TR: int, rank_ab: int) -> int:
    T = TR // rank_ab
    assert TR == T * rank_ab, f"Merged dimension TR={TR} must be divisible by rank_ab={rank_ab}"
    return T


# The decode kernel stages the state tile with an asynchronous copy and waits for it with a time limit; if
# that wait ever ran out it says so in a device word (hdla_recurrent_read_status).  Decode steps are short,
# so the word is fetched (without blocking) only every _POLL_EVERY calls and looked at when the copy has
# landed; check_recurrent_status(wait=True) fetches and inspects it at once.
_POLL_EVERY = 256
_poll = {}        # device index -> dict(calls=int, host=pinned int32[1], event=Event|None)


def _poll_state(dev):
    st = _poll.get(dev.index)
    if st is None:
        st = dict(calls=0, host=torch.zeros(1, dtype=torch.int32).pin_memory(), event=None)
        _poll[dev.index] = st
    return st


def _poll_status(lib, dev) -> None:
    st = _poll_state(dev)
    if st["event"] is not None and st["event"].query():
        st["event"] = None
        if int(st["host"][0]):
            raise RuntimeError("libhdla: a device-side wait ran out in the decode kernel; the results of that call "
                               "are invalid and its final state was not written")
    st["calls"] += 1
    if st["calls"] % _POLL_EVERY == 0 and st["event"] is None and not torch.cuda.is_current_stream_capturing():
        _lib.check(lib.hdla_recurrent_read_status(_lib.ptr(st["host"]), _lib.stream_ptr(dev)),
                   "hdla_recurrent_read_status")
        st["event"] = torch.cuda.Event()
        st["event"].record(torch.cuda.current_stream(dev))


def check_recurrent_status(dev, wait: bool = True) -> None:
    """Fetch the decode kernel's status word for ``dev`` now and raise if a wait ever ran out there."""
    dev = torch.device(dev)
    lib = _lib.load()
    st = _poll_state(dev)
    with torch.cuda.device(dev):
        _lib.check(lib.hdla_recurrent_read_status(_lib.ptr(st["host"]), _lib.stream_ptr(dev)),
                   "hdla_recurrent_read_status")
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(dev))
    st["event"] = ev
    if wait:
        ev.synchronize()
        st["event"] = None
        if int(st["host"][0]):
            raise RuntimeError("libhdla: a device-side wait ran out in the decode kernel")


class FusedRecurrentDPLRDeltaRuleFunction(torch.autograd.Function):
    """Forward only, like the reference (HRDPLR/recurrent.py:180-224)."""

    @staticmethod
    @contiguous
    @autocast_custom_fwd
    def forward(ctx, q, k, v, a, b, gk, rank_ab, scale=None, initial_state=None, output_final_state=False,
                reverse=False, cu_seqlens=None):
        o, ht = fused_recurrent_dplr_delta_rule_fwd(
            q=q, k=k, v=v, a=a, b=b, gk=gk, rank_ab=rank_ab, scale=scale, initial_state=initial_state,
            output_final_state=output_final_state, reverse=reverse, cu_seqlens=cu_seqlens)
        return o, ht

    @staticmethod
    @contiguous
    @autocast_custom_bwd
    def backward(ctx, do, dht):
        raise NotImplementedError(
            "Backward pass for fused_recurrent_dplr_delta_rule is not implemented and will not be supported. "
            "This kernel is only for inference. For training, please use `chunk_hrdplr_delta_rule`.")


def fused_recurrent_dplr_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    a: torch.Tensor,
    b: torch.Tensor,
    gk: torch.Tensor,
    rank_ab: int = 1,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    reverse: bool = False,
    cu_seqlens: Optional[torch.Tensor] = None,
    head_first: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Drop-in for the reference's ``fused_recurrent_dplr_delta_rule`` (HRDPLR/recurrent.py:227-319):
    S_t = diag(exp(gk_t)) S_{t-1} + sum_r b_t^(r) (a_t^(r)^T S_{t-1}) + k_t v_t^T, o_t = scale q_t^T S_t."""
    assert head_first == False, ""
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                f"Please flatten variable-length inputs before processing.")
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}.")
    for name, t in (("a", a), ("b", b)):
        if t.dim() != 4:
            raise ValueError(f"{name} must have 4 dimensions [B, T*RANK_AB, H, K], got {t.dim()}")
    T_expected = _tokens_of_merged(a.shape[1], rank_ab)
    assert q.shape[1] == T_expected, f"q time dimension {q.shape[1]} must match T={T_expected} from merged dimension"
    if scale is None:
        scale = q.shape[-1] ** -0.5
    o, final_state = FusedRecurrentDPLRDeltaRuleFunction.apply(
        q, k, v, a, b, gk, rank_ab, scale, initial_state, output_final_state, reverse, cu_seqlens)
    return o, final_state
