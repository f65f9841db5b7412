"""Context parallelism for long sequences: each rank holds a contiguous slice of T.

The chunked algorithm couples chunks only through the fp32 ``[B,H,K,V]`` state entering a chunk
(reference: the serial loop of HRDPLR/fwd_triton.py:853 forward, HRDPLR/bwd_triton.py:160 backward).
Across ranks that state is the only thing exchanged: rank r receives S from r-1, runs its slice
with ``initial_state = S`` and sends its final state to r+1; in backward the state gradient flows
the other way.  The exchange is point-to-point (``torch.distributed`` send/recv: NCCL over NVLink
on GPUs, gloo on CPU for tests); the received state lands in local memory before any kernel reads it.

The pieces are autograd functions, so the local operator in between is the ordinary
``chunk_hrdplr_delta_rule`` (or, in CPU tests, the oracle).
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


class _RecvStateFromPrev(torch.autograd.Function):
    """forward: rank 0 passes ``state`` through, others receive it from rank-1.
    backward: rank 0 returns the gradient (dh0), others send it to rank-1."""

    @staticmethod
    def forward(ctx, state, group):
        ctx.group = group
        rank = dist.get_rank(group)
        ctx.rank = rank
        if rank == 0:
            return state.clone()
        buf = torch.empty_like(state)
        dist.recv(buf, src=dist.get_global_rank(group, rank - 1) if group is not None else rank - 1, group=group)
        return buf

    @staticmethod
    def backward(ctx, g):
        if ctx.rank == 0:
            return g, None
        dst = dist.get_global_rank(ctx.group, ctx.rank - 1) if ctx.group is not None else ctx.rank - 1
        dist.send(g.contiguous(), dst=dst, group=ctx.group)
        return None, None


class _SendStateToNext(torch.autograd.Function):
    """forward: send the final state to rank+1 (the last rank keeps it).
    backward: add the state gradient received from rank+1 to the local one."""

    @staticmethod
    def forward(ctx, state, group):
        ctx.group = group
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        ctx.rank, ctx.world = rank, world
        if rank < world - 1:
            dst = dist.get_global_rank(group, rank + 1) if group is not None else rank + 1
            dist.send(state.contiguous(), dst=dst, group=group)
        return state.clone()

    @staticmethod
    def backward(ctx, g):
        if ctx.rank < ctx.world - 1:
            buf = torch.empty_like(g)
            src = dist.get_global_rank(ctx.group, ctx.rank + 1) if ctx.group is not None else ctx.rank + 1
            dist.recv(buf, src=src, group=ctx.group)
            g = g + buf
        return g, None


class _Attach(torch.autograd.Function):
    """Ties the sent state into the graph of ``o`` so its backward (the receive) always runs."""

    @staticmethod
    def forward(ctx, o, token):
        ctx.shape, ctx.dtype, ctx.device = token.shape, token.dtype, token.device
        return o.view_as(o)

    @staticmethod
    def backward(ctx, go):
        return go, torch.zeros(ctx.shape, dtype=ctx.dtype, device=ctx.device)


def cp_chunk_hrdplr_delta_rule(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, a: torch.Tensor, b: torch.Tensor, gk: torch.Tensor,
    RANK_AB: int, scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False, chunk_size: int = 64, group=None,
    op: Optional[Callable] = None,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Chunked operator on this rank's T-slice of a sequence sharded over ``group``.

    Arguments are the local slices (``q`` is ``[B, T_local, H, K]`` etc.; ``shard_time`` gives the
    split); ``initial_state`` is used on rank 0 only.  Returns ``(o_local, final_state)`` where
    ``final_state`` is the state after this rank's slice (the sequence's final state on the last
    rank).  ``op`` is the local operator with the signature of ``chunk_hrdplr_delta_rule``; it
    defaults to the CUDA operator of this package."""
    if op is None:
        from .hrdplr import chunk_hrdplr_delta_rule as op
    B, _, H, K = q.shape
    V = v.shape[-1]
    scale = K ** -0.5 if scale is None else scale
    s0 = initial_state
    if s0 is None:
        s0 = torch.zeros(B, H, K, V, dtype=torch.float32, device=q.device)
    s_in = _RecvStateFromPrev.apply(s0, group)
    o, s_out = op(q, k, v, a, b, gk, RANK_AB, scale=scale, initial_state=s_in, output_final_state=True,
                  chunk_size=chunk_size)
    s_sent = _SendStateToNext.apply(s_out, group)
    o = _Attach.apply(o, s_sent)
    return o, (s_sent if output_final_state else None)
