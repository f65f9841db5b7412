"""Operators either side of the HDLA operator in the reference layer.

``parameterize_a_b`` -- the rank-2 (a, b) parametrisation from beta, k and log_f
(reference: HRDPLR/hdla_custom.py:19-43, which computes a and b but never returns them), as one
CUDA kernel forward and one backward (``hdla_param_ab_fwd`` / ``hdla_param_ab_bwd``).

``rms_norm_fused_gate`` -- the layer's output epilogue, RMS norm of ``x * sigmoid(gate)`` over the hidden
row times a weight (reference: RMSNormFusedGate, HRDPLR/normalizations/rms_norm.py:48-91 with
gate_act="sigmoid", gate_pos="pre"), forward and backward kernels ``hdla_norm_gate_fwd`` / ``_bwd``.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib


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
    """``a, b`` of shape ``[B, 2T, H, K]`` (row ``2t + r``) from ``beta [B,T,H,1]``, ``k`` and ``log_f [B,T,H,K]``."""
    return _ParamAB.apply(beta, k, log_f)


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
