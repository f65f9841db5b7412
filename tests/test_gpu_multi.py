"""GPU, 2 ranks over NCCL (skipped with fewer than 2 GPUs): context-parallel forward + backward of
the CUDA operator equals the single-GPU result; batch x head shards need no exchange."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
R = 2


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, T, out, one_gpu=False):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    dev = torch.device("cuda", 0 if one_gpu else rank)
    torch.cuda.set_device(dev)
    if one_gpu:          # ranks sharing one GPU: the maps travel through the host (gloo); no kernel waits for another rank
        dist.init_process_group("gloo", rank=rank, world_size=world)
    else:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import hdla_impl_b200 as H
        from hdla_impl_b200.context_parallel import cp_chunk_hrdplr_delta_rule
        from hdla_impl_b200.sharding import shard_time
        from hdla_impl_b200.synthetic import make_inputs
        from oracle import hdla_oracle as orc
        C = 64
        x = make_inputs(1, T, 2, 128, 128, R, seed=4, dtype=torch.bfloat16, h0_std=0.1, with_dht=True)
        x["gk"] = x["gk"].float()
        names = ("q", "k", "v", "a", "b", "gk")
        lo, hi = shard_time(T, rank, world, C)
        rr = lambda n: R if n in ("a", "b") else 1
        lv = [x[n][:, lo * rr(n):hi * rr(n)].to(dev).requires_grad_(True) for n in names]
        h0 = x["h0"].to(dev).requires_grad_(True)
        o, ht = cp_chunk_hrdplr_delta_rule(*lv, R, initial_state=h0, output_final_state=True, chunk_size=C)
        # every rank's returned final state enters the loss (weights differ per rank)
        dht_r = [x["dht"].to(dev) * (0.5 + r_) for r_ in range(world)]
        loss = (o.float() * x["do"][:, lo:hi].to(dev).float()).sum() + (ht * dht_r[rank]).sum()
        grads = torch.autograd.grad(loss, lv + [h0], allow_unused=True)
        # single-GPU truth on this rank's device: the slices chained through their boundary states, with the same loss
        full = [x[n].to(dev).requires_grad_(True) for n in names]
        h0f = x["h0"].to(dev).requires_grad_(True)
        state, lf, o_parts = h0f, 0.0, []
        for r_ in range(world):
            l_, h_ = shard_time(T, r_, world, C)
            part = [t[:, l_ * rr(n):h_ * rr(n)] for t, n in zip(full, names)]
            o_r, state = H.chunk_hrdplr_delta_rule(*part, R, initial_state=state, output_final_state=True, chunk_size=C)
            lf = lf + (o_r.float() * x["do"][:, l_:h_].to(dev).float()).sum() + (state * dht_r[r_]).sum()
            o_parts.append(o_r)
            if r_ == rank:
                ht_true = state
        of = torch.cat(o_parts, 1)
        gf = torch.autograd.grad(lf, full + [h0f])
        errs = [orc.rel_err(o, of[:, lo:hi]), orc.rel_err(ht, ht_true)]
        for g, gg, n in zip(grads[:6], gf[:6], names):
            errs.append(orc.rel_err(g, gg[:, lo * rr(n):hi * rr(n)]))
        if rank == 0:
            errs.append(orc.rel_err(grads[6], gf[6]))
        else:                                  # initial_state is used on rank 0 only: zero gradient elsewhere
            assert grads[6] is None or float(grads[6].abs().max()) == 0.0
        out[rank] = max(errs)
        HD_check = H.check_status
        HD_check(dev, wait=True)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("T", [512, 4096])      # 4096: 32 chunks per rank, scanned as 4 concurrent segments
def test_context_parallel_two_gpus_matches_one_gpu(T):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), T, out), nprocs=2, join=True)
    # the two paths round the boundary state differently (bf16 checkpoints): bf16 tolerance
    assert len(out) == 2 and max(out.values()) < 2e-2, dict(out)


@pytest.mark.parametrize("world,T", [(2, 512), (3, 4096 + 64 * 3)])
def test_context_parallel_ranks_sharing_one_gpu(world, T):
    """The phased library calls, the composition of the gathered affine state maps and the protocol around them
    (every rank's own final-state gradient, dh0 on rank 0 only) with all ranks as processes on ONE GPU: the maps are
    gathered through the host, so no kernel of one rank ever waits for another rank's.  Same checks as on two GPUs."""
    if torch.cuda.device_count() < 1:
        pytest.skip("needs a GPU")
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), T, out, True), nprocs=world, join=True)
    assert len(out) == world and max(out.values()) < 2e-2, dict(out)
