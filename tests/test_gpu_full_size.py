"""GPU: parity at the benchmark's full sizes.  The oracle is too slow for the whole problem, but
(batch, head) pairs are independent, so one pair of the full-size run is compared with the oracle run
on that pair alone; and the full-size results must not depend on how the batch is cut."""
import pytest
import torch

from oracle import hdla_oracle as orc
from hdla_impl_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu
R = 2
NAMES = ("q", "k", "v", "a", "b", "gk")


def test_cfg1_full_size_slice_against_oracle():
    """B8 T4096 H16 K=V=128 bf16 chunk 64: forward + backward of the whole batch on the GPU; (b, h) = (5, 11)
    against the fp64 oracle; gradients of all inputs within 2e-2."""
    import hdla_impl_b200 as H
    dev = torch.device("cuda:0")
    B, T, Hh, K, V = 8, 4096, 16, 128, 128
    x = make_inputs(B, T, Hh, K, V, R, seed=0, dtype=torch.bfloat16)
    lv = [x[n].to(dev).requires_grad_(True) for n in NAMES]
    o, ht = H.chunk_hrdplr_delta_rule(*lv, R, chunk_size=64, output_final_state=True)
    grads = torch.autograd.grad(o, lv, x["do"].to(dev))
    H.check_status(dev, wait=True)
    b, h = 5, 11
    sl = lambda t: t[b:b + 1, :, h:h + 1].double()
    st = orc.staged_forward(*[sl(x[n]) for n in NAMES], R, K ** -0.5, None, 64)
    g = orc.staged_backward(st, sl(x["do"]), None)
    bad = []
    for name, got, ref in [("o", o, st["o_bthv"]), ("ht", ht[b:b + 1, h:h + 1], st["ht"])] + \
            [(n, t, g[n]) for n, t in zip(("dq", "dk", "dv", "da", "db", "dgk"), grads)]:
        got = got if name == "ht" else got[b:b + 1, :, h:h + 1]
        e = orc.rel_err(got, ref)
        if not e < 2e-2:
            bad.append(f"{name}: {e:.3e}")
    assert not bad, "; ".join(bad)
    # independence of the batch cut: the first five sequences alone (80 (batch, head) pairs: still the one-level scan)
    # give bit-identical results
    lv2 = [x[n][:5].to(dev).requires_grad_(True) for n in NAMES]
    o2, _ = H.chunk_hrdplr_delta_rule(*lv2, R, chunk_size=64)
    g2 = torch.autograd.grad(o2, lv2, x["do"][:5].to(dev))
    assert torch.equal(o2, o[:5])
    for a_, b_ in zip(g2, grads):
        assert torch.equal(a_, b_[:5])
    # the first two alone run the two-level scan (states composed from per-segment maps in fp32): same results to
    # well within the bf16 tolerance, not bit for bit
    lv3 = [x[n][:2].to(dev).requires_grad_(True) for n in NAMES]
    o3, _ = H.chunk_hrdplr_delta_rule(*lv3, R, chunk_size=64)
    g3 = torch.autograd.grad(o3, lv3, x["do"][:2].to(dev))
    assert orc.rel_err(o3, o[:2]) < 5e-3
    for a_, b_ in zip(g3, grads):
        assert orc.rel_err(a_, b_[:2]) < 5e-3


def test_cfg3_full_size_slice_against_oracle():
    """B1 T65536 H16 K=V=128 bf16 chunk 64 on one GPU (1024 chunks per head, scanned as concurrent segments whose
    affine maps are composed in fp32): head 9 -- o, the final state and every gradient, the final state's
    gradient included -- against the fp64 oracle run on that head alone, within 2e-2."""
    import hdla_impl_b200 as H
    dev = torch.device("cuda:0")
    B, T, Hh, K, V = 1, 65536, 16, 128, 128
    x = make_inputs(B, T, Hh, K, V, R, seed=3, dtype=torch.bfloat16, with_dht=True)
    lv = [x[n].to(dev).requires_grad_(True) for n in NAMES]
    o, ht = H.chunk_hrdplr_delta_rule(*lv, R, chunk_size=64, output_final_state=True)
    grads = torch.autograd.grad([o, ht], lv, [x["do"].to(dev), x["dht"].to(dev)])
    H.check_status(dev, wait=True)
    h = 9
    sl = lambda t: t[:, :, h:h + 1].double()
    st = orc.staged_forward(*[sl(x[n]) for n in NAMES], R, K ** -0.5, None, 64)
    g = orc.staged_backward(st, sl(x["do"]), x["dht"][:, h:h + 1].double())
    bad = []
    for name, got, ref in [("o", o[:, :, h:h + 1], st["o_bthv"]), ("ht", ht[:, h:h + 1], st["ht"])] + \
            [(n, t[:, :, h:h + 1], g[n]) for n, t in zip(("dq", "dk", "dv", "da", "db", "dgk"), grads)]:
        e = orc.rel_err(got, ref)
        if not e < 2e-2:
            bad.append(f"{name}: {e:.3e}")
    assert not bad, "; ".join(bad)


def test_cfg2_full_size_decode_against_oracle():
    """256 sequences x 32 heads, K=V=128, bf16 tokens, fp32 state N(0, 0.02): 4 decode steps on the GPU;
    sequences 0 and 200 against the fp64 recurrence."""
    import hdla_impl_b200 as H
    dev = torch.device("cuda:0")
    B, Hh, K, V, steps = 256, 32, 128, 128, 4
    x = make_inputs(B, steps, Hh, K, V, R, seed=2, dtype=torch.bfloat16, h0_std=0.02)
    S = x["h0"].to(dev).clone()
    outs = []
    for t in range(steps):
        cur = [x[n][:, t * (R if n in ("a", "b") else 1):(t + 1) * (R if n in ("a", "b") else 1)].to(dev) for n in NAMES]
        o, S = H.fused_recurrent_dplr_delta_rule_fwd(*cur, R, K ** -0.5, S, True, inplace_state=True)
        outs.append(o)
    o = torch.cat(outs, 1)
    for s in (0, 200):
        ro, rh = orc.recurrent_ref(*[x[n][s:s + 1].double() for n in NAMES], R, None, x["h0"][s:s + 1])
        assert orc.rel_err(o[s:s + 1], ro) < 2e-2
        assert orc.rel_err(S[s:s + 1], rh) < 1e-3
