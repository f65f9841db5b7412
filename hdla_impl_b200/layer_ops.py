"""Operators either side of the HDLA operator in the reference layer.

``parameterize_a_b`` -- the rank-2 (a, b) parametrisation from beta, k and log_f
(reference: HRDPLR/hdla_custom.py:19-43, which computes a and b but never returns them), as one
CUDA kernel forward and one backward (``hdla_param_ab_fwd`` / ``hdla_param_ab_bwd``).

``chunk_hdla_delta_rule`` -- the layer's pair of calls ``parameterize_a_b`` + ``chunk_hrdplr_delta_rule``
(reference: HRDPLR/hdla_custom.py:290-309) as ONE operator call: the operator's chunk-preparation kernel forms
a and b from beta, k and log_f on the way to its operand tiles (``HDLA_FLAG_PARAM_AB``), so a and b are never
written or read and the operator's input is 4 tensors of ``[B,T,H,K]`` plus beta instead of 8.

``rms_norm_fused_gate`` -- the layer's output epilogue, RMS norm of ``x * sigmoid(gate)`` over the hidden
row times a weight (reference: RMSNormFusedGate, HRDPLR/normalizations/rms_norm.py:48-91 with
gate_act="sigmoid", gate_pos="pre"), forward and backward kernels ``hdla_norm_gate_fwd`` / ``_bwd``.
"""
from __future__ import annotations

import ctypes as C
import warnings
from typing import Optional, Tuple

import torch

from . import _lib
from . import hrdplr as _op


class _ParamAB(torch.autograd.Function):
    @staticmethod
    def forward(ctx, beta, k, log_f):
        dev = _lib.require_cuda(beta, k, log_f)
        B, T, H, K = k.shape
        if beta.shape != (B, T, H, 1) or log_f.shape != k.shape:
            raise ValueError(f"beta {tuple(beta.shape)} must be [B,T,H,1] and log_f {tuple(log_f.shape)} like k {tuple(k.shape)}")
        dt = k.dtype
        beta, k, log_f = beta.to(dt).contiguous(), k.contiguous(), log_f.to(dt).contiguous()
        with torch.cuda.device(dev):
            a = torch.empty(B, 2 * T, H, K, dtype=dt, device=dev)
            b = torch.empty_like(a)
            rc = _lib.load().hdla_param_ab_fwd(_lib.ptr(beta), _lib.ptr(k), _lib.ptr(log_f), _lib.ptr(a), _lib.ptr(b),
                                               B, T, H, K, _lib.dtype_code(dt), _lib.stream_ptr(dev))
        _lib.check(rc, "hdla_param_ab_fwd")
        ctx.save_for_backward(beta, k, log_f)
        return a, b

    @staticmethod
    def backward(ctx, da, db):
        beta, k, log_f = ctx.saved_tensors
        dev = k.device
        B, T, H, K = k.shape
        da, db = da.contiguous().to(k.dtype), db.contiguous().to(k.dtype)
        with torch.cuda.device(dev):
            dbeta, dk, dlog_f = torch.empty_like(beta), torch.empty_like(k), torch.empty_like(log_f)
            rc = _lib.load().hdla_param_ab_bwd(_lib.ptr(beta), _lib.ptr(k), _lib.ptr(log_f), _lib.ptr(da), _lib.ptr(db),
                                               _lib.ptr(dbeta), _lib.ptr(dk), _lib.ptr(dlog_f), B, T, H, K,
                                               _lib.dtype_code(k.dtype), _lib.stream_ptr(dev))
        _lib.check(rc, "hdla_param_ab_bwd")
        return dbeta, dk, dlog_f


def parameterize_a_b(beta: torch.Tensor, k: torch.Tensor, log_f: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``a, b`` of shape ``[B, 2T, H, K]`` (row ``2t + r``) from ``beta [B,T,H,1]``, ``k`` and ``log_f [B,T,H,K]``.
    ``beta`` may be a number (the layer uses the constant 2 when it has no beta projection, HRDPLR/hdla_custom.py:226)."""
    if not torch.is_tensor(beta):
        beta = k.new_full(tuple(k.shape[:3]) + (1,), float(beta))
    return _ParamAB.apply(beta, k, log_f)


class _DecayOverflow(Exception):
    """A chunk's total log decay is beyond the bf16 tensor-core pipeline: the caller takes the two-call route."""


class _ChunkHdla(torch.autograd.Function):
    """Operator call with the in-operator a/b parametrisation; gradients for q, k, v, beta, log_f and the state."""

    @staticmethod
    @_op.contiguous
    @_op.autocast_custom_fwd
    def forward(ctx, q, k, v, beta, log_f, scale, initial_state, output_final_state, cu_seqlens, normalize_k=False):
        dev = _lib.require_cuda(q, k, v, beta, log_f, initial_state)
        _op.check_status(dev)
        lib = _lib.load()
        B, T, H, K = q.shape
        V = v.shape[-1]
        N = None if cu_seqlens is None else len(cu_seqlens) - 1
        beta_c = beta.to(q.dtype).contiguous()
        keep = _op.save_workspace_default() and any(
            isinstance(t, torch.Tensor) and t.requires_grad for t in (q, k, v, beta, log_f, initial_state))
        ctx.flags = _lib.FLAG_PARAM_AB | (_lib.FLAG_NORM_K if normalize_k else 0)
        dims = _op._dims(q, v, beta_c, log_f, 2, 64, ctx.flags, cu_seqlens)
        h0 = None if initial_state is None else initial_state.to(torch.float32).contiguous()
        with torch.cuda.device(dev):
            ws = _op._alloc_ws(_op.workspace_bytes(dims, keep), dev)
            o = torch.empty_like(v)
            ht = torch.empty(B if N is None else N, H, K, V, dtype=torch.float32, device=dev) if output_final_state else None
            rc = lib.hdla_chunk_fwd(C.byref(dims), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(beta_c), None,
                                    _lib.ptr(log_f), float(scale), _lib.ptr(h0), _lib.ptr(o), _lib.ptr(ht),
                                    _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
            _lib.check(rc, "hdla_chunk_fwd")
            slot = _op._post_status(ws, dev)
            if _op._overflow_plausible(dev):
                words = _op._wait_words(dev, slot)
                if words[1] and not words[0]:
                    raise _DecayOverflow()
                if words[0] or words[1]:
                    _op._raise_status(words)
        ctx.ws = ws if keep else None
        ctx.cu_seqlens, ctx.scale, ctx.beta_like = cu_seqlens, scale, (beta.shape, beta.dtype)
        ctx.save_for_backward(q, k, v, beta_c, log_f, initial_state)
        return o, ht

    @staticmethod
    @_op.contiguous
    @_op.autocast_custom_bwd
    def backward(ctx, do, dht):
        q, k, v, beta, log_f, initial_state = ctx.saved_tensors
        dev = q.device
        _op.check_status(dev)
        lib = _lib.load()
        ws, ctx.ws = ctx.ws, None
        flags = ctx.flags | (_lib.FLAG_WS_HOLDS_FWD if ws is not None else 0)
        dims = _op._dims(q, v, beta, log_f, 2, 64, flags, ctx.cu_seqlens)
        h0 = None if initial_state is None else initial_state.to(torch.float32).contiguous()
        if do.dtype != q.dtype:
            do = do.to(q.dtype)
        if dht is not None:
            dht = dht.to(torch.float32).contiguous()
        with torch.cuda.device(dev):
            if ws is None:
                ws = _op._alloc_ws(_op.workspace_bytes(dims, True), dev)
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
            dbeta, dlog_f = torch.empty_like(beta), torch.empty_like(log_f)
            dh0 = torch.empty_like(h0) if h0 is not None else None
            rc = lib.hdla_chunk_bwd(C.byref(dims), _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(beta), None,
                                    _lib.ptr(log_f), float(ctx.scale), _lib.ptr(h0), _lib.ptr(do), _lib.ptr(dht),
                                    _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv), _lib.ptr(dbeta), None,
                                    _lib.ptr(dlog_f), _lib.ptr(dh0), _lib.ptr(ws), ws.numel(), _lib.stream_ptr(dev))
            _lib.check(rc, "hdla_chunk_bwd")
            _op._post_status(ws, dev)
        if dh0 is not None and initial_state.dtype != torch.float32:
            dh0 = dh0.to(initial_state.dtype)
        shape, dtype = ctx.beta_like
        return dq, dk, dv, dbeta.view(shape).to(dtype), dlog_f, None, dh0, None, None, None


_warned_two_call = False
L2_NORM_EPS = 1e-5      # of the reference's l2_norm (HRDPLR/normalizations/l2_norm.py:4)


@torch.compiler.disable
def chunk_hdla_delta_rule(
    q: torch.Tensor,       # [B, T, H, K]
    k: torch.Tensor,       # [B, T, H, K]
    v: torch.Tensor,       # [B, T, H, V]
    beta,                  # [B, T, H, 1] or [B, T, H] tensor, or a number
    log_f: torch.Tensor,   # [B, T, H, K]  log decay (the operator's gk)
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    cu_seqlens=None,
    normalize_k: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """What the reference layer computes with ``a, b = parameterize_a_b(beta, k, log_f)`` followed by
    ``chunk_hrdplr_delta_rule(q, k, v, a, b, gk=log_f, RANK_AB=2, ...)`` (HRDPLR/hdla_custom.py:290-309), as one
    operator call on the bf16 tensor-core pipeline.  With ``normalize_k`` the layer's ``k = l2_norm(k)``
    (HRDPLR/hdla_custom.py:248: ``k / sqrt(sum_K k^2 + 1e-5)``) happens inside the operator too and ``k`` is the
    un-normalised tensor.  Problems outside that pipeline (fp32, other head dims, decays beyond its range) take
    the separate calls."""
    global _warned_two_call
    B, T, H, K = q.shape
    if not torch.is_tensor(beta):            # the layer's constant beta = 2 (no beta projection)
        beta = q.new_full((B, T, H, 1), float(beta))
    if k.shape != q.shape or log_f.shape != q.shape or v.shape[:3] != q.shape[:3]:
        raise ValueError(f"k {tuple(k.shape)} and log_f {tuple(log_f.shape)} must match q {tuple(q.shape)}, v "
                         f"{tuple(v.shape)} must be [B, T, H, V]")
    if beta.numel() != B * T * H or beta.shape[:3] != (B, T, H):
        raise ValueError(f"beta {tuple(beta.shape)} must be [B, T, H, 1] or [B, T, H]")
    scale = K ** -0.5 if scale is None else scale
    offsets = _op._seq_offsets(cu_seqlens)
    n_states = B if offsets is None else len(offsets) - 1
    if initial_state is not None and tuple(initial_state.shape) != (n_states, H, K, v.shape[-1]):
        raise ValueError(f"initial_state {tuple(initial_state.shape)} must be [{n_states}, H, K, V] = "
                         f"{(n_states, H, K, v.shape[-1])}")
    if _op._packed_supported(q, v, 2) and log_f.dtype in (torch.bfloat16, torch.float32):
        if offsets is not None and (q.shape[0] != 1 or offsets[0] != 0 or offsets[-1] != T
                                    or any(y < x for x, y in zip(offsets, offsets[1:]))):
            raise ValueError(f"cu_seqlens {offsets} must rise from 0 to T={T} in a batch of one")
        try:
            return _ChunkHdla.apply(q, k, v, beta, log_f, scale, initial_state, output_final_state, offsets,
                                    normalize_k)
        except _DecayOverflow:
            if not _warned_two_call:
                _warned_two_call = True
                warnings.warn("hdla_impl_b200: a chunk's total log decay exceeds what the bf16 tensor-core pipeline "
                              "represents; such calls take parameterize_a_b + the fp32 CUDA-core pipeline "
                              "(correct, much slower)", RuntimeWarning, stacklevel=2)
    if normalize_k:
        kf = k.float()
        k = (kf * torch.rsqrt((kf * kf).sum(-1, keepdim=True) + L2_NORM_EPS)).to(k.dtype)
    a, b = parameterize_a_b(beta.reshape(B, T, H, 1), k, log_f)
    return _op.chunk_hrdplr_delta_rule(q, k, v, a, b, log_f, 2, scale=scale, initial_state=initial_state,
                                       output_final_state=output_final_state, chunk_size=64, cu_seqlens=cu_seqlens)


class _NormGate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, weight, eps):
        dev = _lib.require_cuda(x, gate, weight)
        D = x.shape[-1]
        if gate.shape != x.shape or weight.shape != (D,):
            raise ValueError("gate must be shaped like x and weight like its last dimension")
        dt = x.dtype
        x2, g2, w = x.contiguous(), gate.to(dt).contiguous(), weight.to(dt).contiguous()
        rows = x2.numel() // D
        with torch.cuda.device(dev):
            o = torch.empty_like(x2)
            rc = _lib.load().hdla_norm_gate_fwd(_lib.ptr(x2), _lib.ptr(g2), _lib.ptr(w), _lib.ptr(o), rows, D,
                                                float(eps), _lib.dtype_code(dt), _lib.stream_ptr(dev))
        _lib.check(rc, "hdla_norm_gate_fwd")
        ctx.save_for_backward(x2, g2, w)
        ctx.eps, ctx.wdtype = eps, weight.dtype
        return o

    @staticmethod
    def backward(ctx, do):
        x, gate, w = ctx.saved_tensors
        dev = x.device
        D = x.shape[-1]
        rows = x.numel() // D
        do = do.contiguous().to(x.dtype)
        with torch.cuda.device(dev):
            dx, dg = torch.empty_like(x), torch.empty_like(gate)
            dw = torch.zeros(D, dtype=torch.float32, device=dev)
            rc = _lib.load().hdla_norm_gate_bwd(_lib.ptr(x), _lib.ptr(gate), _lib.ptr(w), _lib.ptr(do), _lib.ptr(dx),
                                                _lib.ptr(dg), _lib.ptr(dw), rows, D, float(ctx.eps),
                                                _lib.dtype_code(x.dtype), _lib.stream_ptr(dev))
        _lib.check(rc, "hdla_norm_gate_bwd")
        return dx, dg, dw.to(ctx.wdtype), None


def rms_norm_fused_gate(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """``sqrt(D) * y / sqrt(sum(y^2) + eps) * weight`` with ``y = x * sigmoid(gate)`` over the last dimension."""
    return _NormGate.apply(x, gate, weight, eps)
