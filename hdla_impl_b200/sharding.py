"""Partitioning of the operator over the GPUs of one node.

The reference has no multi-GPU code; its kernels put ``B*H`` on the last grid axis
(e.g. HRDPLR/fwd_func.py:45, :253) because (batch, head) pairs never interact.  That independence
is what is sharded here: each rank owns a contiguous block of the flattened ``B x H`` pairs and no
collective touches the data path.  Sequences too long for that (B = 1) are sharded over time
instead -- see ``context_parallel.py``.
"""
from __future__ import annotations

from typing import Tuple


def shard_batch_heads(B: int, H: int, rank: int, world: int) -> Tuple[int, int, int, int]:
    """Return ``(b_lo, b_hi, h_lo, h_hi)``: the batch rows and heads rank ``rank`` of ``world`` owns.

    Ranks split the batch while ``world <= B`` (``B % world == 0``); beyond that every batch row is
    split over ``world // B`` ranks by head (``world % B == 0`` and ``H % (world // B) == 0``).
    """
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if world <= B:
        if B % world:
            raise ValueError(f"batch {B} is not divisible by {world} ranks")
        per = B // world
        return rank * per, (rank + 1) * per, 0, H
    if world % B:
        raise ValueError(f"{world} ranks cannot split batch {B} evenly")
    per_row = world // B
    if H % per_row:
        raise ValueError(f"{H} heads are not divisible by {per_row} ranks per batch row")
    hp = H // per_row
    b = rank // per_row
    j = rank % per_row
    return b, b + 1, j * hp, (j + 1) * hp


def shard_time(T: int, rank: int, world: int, chunk: int) -> Tuple[int, int]:
    """Contiguous, chunk-aligned token range ``[t_lo, t_hi)`` of rank ``rank`` for context parallelism.

    Whole chunks are dealt out as evenly as possible (earlier ranks take the remainder); the last
    rank also takes a ragged final chunk."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    nt = (T + chunk - 1) // chunk
    base, rem = divmod(nt, world)
    lo_c = rank * base + min(rank, rem)
    hi_c = lo_c + base + (1 if rank < rem else 0)
    return min(lo_c * chunk, T), min(hi_c * chunk, T)
