"""Context parallelism for long sequences: each rank holds a contiguous slice of T.

The chunked algorithm couples chunks only through the fp32 ``[B,H,K,V]`` state entering a chunk
(reference: the serial loop of HRDPLR/fwd_triton.py:853 forward, HRDPLR/bwd_triton.py:160 backward).
Across ranks that state is the only thing exchanged: rank r receives S from r-1, runs its slice
with ``initial_state = S`` and sends its final state to r+1; in backward the state gradient flows
the other way.  The exchange is point-to-point (``torch.distributed`` send/recv: NCCL over NVLink
on GPUs, gloo on CPU for tests); the received state lands in local memory before any kernel reads it.

Two forms are provided.  The generic one strings autograd send/recv functions around the ordinary
local operator (any ``op``; used on CPU with the oracle): rank r waits for rank r-1.  The fused one
(``_CPChunkFunction``, bf16 CUDA path) uses the library's phased calls so that all ranks scan at the
same time and exchange one all-gather of affine state maps per direction.
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


def _compose(lib, dims, T, F, S0, pre, post, out, count, t_stride, f_stride, reverse, dev):
    import ctypes as C
    from . import _lib
    rc = lib.hdla_compose_states(C.byref(dims), _lib.ptr(T), _lib.ptr(F), _lib.ptr(S0), _lib.ptr(pre), _lib.ptr(post),
                                 _lib.ptr(out), int(count), int(t_stride), int(f_stride), int(reverse),
                                 _lib.stream_ptr(dev))
    _lib.check(rc, "hdla_compose_states")


def _all_gather_maps(out: torch.Tensor, mine: torch.Tensor, group) -> None:
    """``out[r] = mine of rank r``.  NCCL groups gather on the device; a group whose backend cannot take CUDA tensors
    (gloo: ranks that share one GPU in tests, or hosts without NCCL) is served through host memory."""
    if dist.get_backend(group) == "nccl":
        dist.all_gather_into_tensor(out, mine, group=group)
        return
    host = mine.detach().cpu()
    parts = [torch.empty_like(host) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, host, group=group)
    out.copy_(torch.stack(parts).to(out.device, non_blocking=False))


class _CPChunkFunction(torch.autograd.Function):
    """Context-parallel chunked operator on the CUDA library, with the scans of all ranks running
    concurrently.

    The state leaving a rank is affine in the state entering it, ``S_out = T S_in + F``: ``T`` is the
    product of the chunk transition matrices (one scan of a K x K identity, ``HDLA_PHASE_TRANSITION``)
    and ``F`` the state reached from zero (``HDLA_PHASE_STATE``).  Every rank computes its ``(T, F)``
    at the same time, one all-gather distributes them, each rank composes the state entering its slice
    locally (``hdla_compose_states``, one launch) and only then runs the real scan (``HDLA_PHASE_POST``).
    Backward is the mirror image with ``T^T``; every rank contributes the gradient of its own returned
    final state.  Per rank the scan work is three passes over T/world chunks instead of one pass over T.
    """

    @staticmethod
    def forward(ctx, q, k, v, a, b, gk, scale, initial_state, RANK_AB, chunk_size, group):
        import ctypes as C
        from . import _lib
        from .hrdplr import _alloc_ws, _dims, _post_status, check_status, workspace_bytes
        q, k, v, a, b, gk = (t.contiguous() for t in (q, k, v, a, b, gk))
        dev = q.device
        rank, world = dist.get_rank(group), dist.get_world_size(group)
        B, T, H, K = q.shape
        V = v.shape[-1]
        lib = _lib.load()
        check_status(dev)
        # one dims structure, its flags rewritten per phase, and the tensor / stream pointers taken once: a step makes
        # a dozen calls into the library and their host-side cost adds up to the step's critical path
        d = _dims(q, v, a, gk, RANK_AB, chunk_size)
        base_flags = d.flags
        ws = _alloc_ws(workspace_bytes(d, True), dev)
        f32 = dict(dtype=torch.float32, device=dev)
        ins = [_lib.ptr(t) for t in (q, k, v, a, b, gk)]
        ws_p, ws_n, sc = _lib.ptr(ws), ws.numel(), float(scale)

        def fwd(phase, h0, o, ht):
            d.flags = base_flags | phase
            rc = lib.hdla_chunk_fwd(C.byref(d), *ins, sc, _lib.ptr(h0), _lib.ptr(o), _lib.ptr(ht), ws_p, ws_n, stream)
            if rc:
                _lib.check(rc, "hdla_chunk_fwd")

        def mk(_phase):
            d.flags = base_flags
            return d

        with torch.cuda.device(dev):
            stream = _lib.stream_ptr(dev)
            fwd(_lib.PHASE_PRE, None, None, None)
            # one collective per direction: every rank contributes its transition map, its state-from-zero map and
            # (rank 0 only) the sequence's initial state, packed as [3, B, H, K, V] (K == V on this path)
            pack = torch.empty(3, B, H, K, V, **f32)
            fwd(_lib.PHASE_TRANSITION, None, None, pack[0])
            fwd(_lib.PHASE_STATE, None, None, pack[1])
            if rank == 0 and initial_state is not None:
                pack[2].copy_(initial_state)
            else:
                pack[2].zero_()
            maps = torch.empty(world, 3, B, H, K, V, **f32)
            _all_gather_maps(maps, pack, group)
            # state entering this rank's slice: the maps of ranks 0 .. rank-1 applied to the initial state
            S = torch.empty(B, H, K, V, **f32)
            _compose(lib, mk(0), maps[0, 0], maps[0, 1], maps[0, 2], None, None, S, rank, 3 * B * H, 3 * B * H, 0, dev)
            o = torch.empty_like(v)
            ht = torch.empty(B, H, K, V, **f32)
            fwd(_lib.PHASE_POST, S, o, ht)
            _post_status(ws, dev)
        ctx.save_for_backward(q, k, v, a, b, gk, S, maps)
        ctx.ws, ctx.scale, ctx.R, ctx.chunk, ctx.group = ws, scale, RANK_AB, chunk_size, group
        ctx.has_h0 = initial_state is not None
        ctx.rank, ctx.world = rank, world
        return o, ht

    @staticmethod
    def backward(ctx, do, dht):
        import ctypes as C
        from . import _lib
        from .hrdplr import _dims, _post_status, check_status
        q, k, v, a, b, gk, S_in, maps = ctx.saved_tensors
        group = ctx.group
        dev = q.device
        rank, world = ctx.rank, ctx.world
        B, T, H, K = q.shape
        V = v.shape[-1]
        lib = _lib.load()
        check_status(dev)
        ws = ctx.ws
        ctx.ws = None
        do = do.contiguous().to(q.dtype)
        f32 = dict(dtype=torch.float32, device=dev)
        grads = [torch.empty_like(t) for t in (q, k, v, a, b, gk)]
        d = _dims(q, v, a, gk, ctx.R, ctx.chunk, _lib.FLAG_WS_HOLDS_FWD)
        base_flags = d.flags
        ins = [_lib.ptr(t) for t in (q, k, v, a, b, gk)]
        gp, none6 = [_lib.ptr(t) for t in grads], [None] * 6
        ws_p, ws_n, sc, s_in, do_p = _lib.ptr(ws), ws.numel(), float(ctx.scale), _lib.ptr(S_in), _lib.ptr(do)

        def bwd(phase, dht_, dh0_, with_grads):
            d.flags = base_flags | phase
            rc = lib.hdla_chunk_bwd(C.byref(d), *ins, sc, s_in, do_p, _lib.ptr(dht_), *(gp if with_grads else none6),
                                    _lib.ptr(dh0_), ws_p, ws_n, stream)
            if rc:
                _lib.check(rc, "hdla_chunk_bwd")

        def mk(_phase):
            d.flags = base_flags & ~_lib.FLAG_WS_HOLDS_FWD
            return d

        with torch.cuda.device(dev):
            stream = _lib.stream_ptr(dev)
            bwd(_lib.PHASE_PRE, None, None, False)
            # mirror image: every rank contributes its gradient-from-zero map G and the gradient of the final
            # state IT returned (rank j's final state is the state entering rank j+1)
            pack = torch.empty(2, B, H, K, V, **f32)
            bwd(_lib.PHASE_STATE, None, pack[0], False)
            if dht is not None:
                pack[1].copy_(dht)
            else:
                pack[1].zero_()
            gmaps = torch.empty(world, 2, B, H, K, V, **f32)
            _all_gather_maps(gmaps, pack, group)
            # gradient of the state leaving this rank: dht_rank + E_{rank+1}, with E_j = T_j^T (dht_j + E_{j+1}) + G_j
            # the gradient of the state entering rank j (E_world = 0)
            D = torch.empty(B, H, K, V, **f32)
            n_after = world - 1 - rank
            nxt = min(rank + 1, world - 1)
            _compose(lib, mk(0), maps[nxt, 0], gmaps[nxt, 0], None, gmaps[nxt, 1], gmaps[rank, 1], D, n_after,
                     3 * B * H, 2 * B * H, 1, dev)
            dh0 = torch.empty(B, H, K, V, **f32)
            bwd(_lib.PHASE_POST, D, dh0, True)
            _post_status(ws, dev)
        dq, dk, dv, da, db, dgk = grads
        # the gradient of the state entering this slice is the sequence's dh0 on rank 0 only (initial_state is
        # used there alone); elsewhere the argument was ignored and gets a zero gradient
        if not ctx.has_h0:
            dh0 = None
        elif rank != 0:
            dh0 = torch.zeros_like(dh0)
        return dq, dk, dv, da, db, dgk, None, dh0, None, None, None


def _fused_supported(q, v, gk, RANK_AB, chunk_size) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and RANK_AB == 2 and q.shape[-1] == 128 and v.shape[-1] == 128
            and chunk_size >= 64 and q.shape[1] >= 64)


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
    if op is None and _fused_supported(q, v, gk, RANK_AB, chunk_size) and chunk_size == 64:
        scale_ = q.shape[-1] ** -0.5 if scale is None else scale
        o, ht = _CPChunkFunction.apply(q, k, v, a, b, gk, scale_, initial_state, RANK_AB, chunk_size, group)
        return o, (ht if output_final_state else None)
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
