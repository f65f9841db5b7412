"""CPU, gloo, world_size 2 and 3: batch x head sharding and the context-parallel state hand-off.
The chunk maths is done by the oracle (there is no CPU path in the product); what is tested is
the host-side partitioning and the send/recv plumbing with autograd."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hdla_impl_b200.sharding import shard_batch_heads, shard_time

R = 2


def test_shard_batch_heads_covers_everything_once():
    for B, H, world in [(8, 16, 1), (8, 16, 2), (8, 16, 8), (8, 16, 16), (1, 16, 8), (2, 4, 8), (4, 6, 2)]:
        seen = set()
        for r in range(world):
            b0, b1, h0, h1 = shard_batch_heads(B, H, r, world)
            for bb in range(b0, b1):
                for hh in range(h0, h1):
                    assert (bb, hh) not in seen
                    seen.add((bb, hh))
        assert len(seen) == B * H
    with pytest.raises(ValueError):
        shard_batch_heads(3, 4, 0, 2)
    with pytest.raises(ValueError):
        shard_batch_heads(1, 6, 0, 4)
    with pytest.raises(ValueError):
        shard_batch_heads(8, 16, 8, 8)


def test_shard_time_is_contiguous_and_chunk_aligned():
    for T, world, C in [(65536, 8, 64), (1000, 3, 64), (64, 4, 64), (100, 2, 16)]:
        prev = 0
        for r in range(world):
            lo, hi = shard_time(T, r, world, C)
            assert lo == prev and lo % C == 0 and hi >= lo
            prev = hi
        assert prev == T


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _oracle_op(q, k, v, a, b, gk, RANK_AB, scale=None, initial_state=None, output_final_state=True, chunk_size=64):
    from oracle import hdla_oracle as orc
    return orc.chunked_ref(q, k, v, a, b, gk, RANK_AB, scale, initial_state, output_final_state, chunk_size)


def _cp_worker(rank, world, port, T, C, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hdla_impl_b200.context_parallel import cp_chunk_hrdplr_delta_rule
        from hdla_impl_b200.synthetic import make_inputs
        from oracle import hdla_oracle as orc
        torch.set_num_threads(1)
        x = make_inputs(1, T, 2, 16, 16, R, seed=3, gk_div=4.0, h0_std=0.5, with_dht=True)
        lo, hi = shard_time(T, rank, world, C)
        sl = lambda n, r=1: x[n][:, lo * r:hi * r].double().requires_grad_(True)
        lv = [sl("q"), sl("k"), sl("v"), sl("a", R), sl("b", R), sl("gk")]
        h0 = x["h0"].double().requires_grad_(True)
        o, ht = cp_chunk_hrdplr_delta_rule(*lv, R, scale=0.3, initial_state=h0, output_final_state=True,
                                           chunk_size=C, op=_oracle_op)
        loss = (o * x["do"][:, lo:hi].double()).sum()
        if rank == world - 1:
            loss = loss + (ht * x["dht"].double()).sum()
        grads = torch.autograd.grad(loss, lv + [h0], allow_unused=True)
        # single-process truth
        fn = lambda q, k, v, a, b, gk, s: orc.chunked_ref(q, k, v, a, b, gk, R, 0.3, s, True, C)
        ro, rh, rg = orc.autograd_ref(fn, x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], x["h0"], x["do"], x["dht"])
        errs = [orc.rel_err(o, ro[:, lo:hi])]
        for g, n, r in zip(grads[:6], ["dq", "dk", "dv", "da", "db", "dgk"], [1, 1, 1, R, R, 1]):
            errs.append(orc.rel_err(g, rg[n][:, lo * r:hi * r]))
        if rank == world - 1:
            errs.append(orc.rel_err(ht, rh))
        if rank == 0:
            errs.append(orc.rel_err(grads[6], rg["dh0"]))
        out[rank] = max(errs)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,T,C", [(2, 96, 16), (3, 80, 16)])
def test_context_parallel_state_handoff_matches_single_process(world, T, C):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_cp_worker, args=(world, _free_port(), T, C, out), nprocs=world, join=True)
    assert len(out) == world
    assert max(out.values()) < 1e-10, dict(out)


def _bh_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hdla_impl_b200.synthetic import make_inputs
        from oracle import hdla_oracle as orc
        torch.set_num_threads(1)
        B, H = 2, 4
        x = make_inputs(B, 32, H, 16, 16, R, seed=1)
        b0, b1, h0, h1 = shard_batch_heads(B, H, rank, world)
        sl = lambda n: x[n][b0:b1, :, h0:h1]
        o, _ = orc.chunked_ref(sl("q"), sl("k"), sl("v"), sl("a"), sl("b"), sl("gk"), R, None, None, False, 16)
        full, _ = orc.chunked_ref(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, None, None, False, 16)
        # the shards need no exchange: gather only to compare
        gathered = [None] * world
        dist.all_gather_object(gathered, (b0, b1, h0, h1, o))
        if rank == 0:
            rec = torch.zeros_like(full)
            for (x0, x1, y0, y1, oo) in gathered:
                rec[x0:x1, :, y0:y1] = oo
            out["err"] = orc.rel_err(rec, full)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_batch_head_shards_reassemble(world):
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_bh_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out["err"] < 1e-12


def _peer_loss_worker(rank, world, port, out):
    """Rank 1 leaves right after the rendezvous, between steps and with nothing in flight; the others run one
    context-parallel forward + backward and must get an error from their send/recv, not a hang."""
    import datetime
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    if rank == 1:
        out[rank] = "left"
        os._exit(0)                                   # no destroy_process_group: the peer is simply gone
    from hdla_impl_b200.context_parallel import cp_chunk_hrdplr_delta_rule
    from hdla_impl_b200.synthetic import make_inputs
    torch.set_num_threads(1)
    T, C = 96, 16
    x = make_inputs(1, T, 1, 16, 16, R, seed=5, gk_div=4.0)
    lo, hi = shard_time(T, rank, world, C)
    sl = lambda n, r=1: x[n][:, lo * r:hi * r].double().requires_grad_(True)
    lv = [sl("q"), sl("k"), sl("v"), sl("a", R), sl("b", R), sl("gk")]
    try:
        o, _ = cp_chunk_hrdplr_delta_rule(*lv, R, scale=0.3, chunk_size=C, op=_oracle_op)
        torch.autograd.grad(o.sum(), lv)
        out[rank] = "completed"
    except Exception as e:                            # gloo reports a closed connection or a timed-out recv
        out[rank] = f"error: {type(e).__name__}: {str(e)[:200]}"
    os._exit(0)                                       # a clean shutdown handshake with a missing peer would block


@pytest.mark.timeout(180)
def test_context_parallel_peer_loss_is_an_error_not_a_hang():
    world = 3
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_peer_loss_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert out[1] == "left"
    # rank 2 waits for a state that never comes; rank 0's send or its backward recv meets the closed peer
    assert out[2].startswith("error"), dict(out)
    assert out[0].startswith("error"), dict(out)


def _gather_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from hdla_impl_b200.context_parallel import _all_gather_maps
        mine = torch.full((3, 2, 4), float(rank + 1))
        got = torch.zeros(world, 3, 2, 4)
        _all_gather_maps(got, mine, None)
        out[rank] = bool(all(torch.equal(got[r], torch.full((3, 2, 4), float(r + 1))) for r in range(world)))
    finally:
        dist.destroy_process_group()


def test_state_map_gather_through_the_host_for_non_nccl_groups():
    """The context-parallel path's one collective per direction, on a group whose backend cannot take device tensors:
    every rank ends up with every rank's maps in rank order."""
    world = 3
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_gather_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    assert len(out) == world and all(out.values())
