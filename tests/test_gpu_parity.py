"""GPU parity: the CUDA operator (through the public entry points, which call the C ABI) against
the fp64 CPU oracle and the golden vectors of the reference's naive implementation.

Tolerances (max|x-ref| / max|ref| per tensor): fp32 inputs 1e-4, bf16 inputs 2e-2.
"""
import os

import numpy as np
import pytest
import torch

from oracle import hdla_oracle as orc
from hdla_impl_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu

R = 2
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2}
GRADS = ["dq", "dk", "dv", "da", "db", "dgk"]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a CUDA device"
    return torch.device("cuda:0")


def run_chunk(x, dev, scale, chunk, use_h0, use_dht, dtype):
    import hdla_impl_b200 as H
    names = ["q", "k", "v", "a", "b", "gk"]
    leaves = [x[n].to(dev).to(dtype if n != "gk" else x[n].dtype).requires_grad_(True) for n in names]
    h0 = x["h0"].to(dev).requires_grad_(True) if use_h0 else None
    o, ht = H.chunk_hrdplr_delta_rule(*leaves, R, scale=scale, initial_state=h0, output_final_state=True,
                                      chunk_size=chunk)
    loss = (o.float() * x["do"].to(dev).float()).sum()
    if use_dht:
        loss = loss + (ht * x["dht"].to(dev)).sum()
    ins = leaves + ([h0] if use_h0 else [])
    grads = torch.autograd.grad(loss, ins)
    out = dict(o=o, ht=ht)
    out.update(dict(zip(GRADS + (["dh0"] if use_h0 else []), grads)))
    return out


def oracle_chunk(x, scale, use_h0, use_dht, dtype):
    """fp64 oracle on the inputs as the device sees them (rounded to `dtype`)."""
    rd = lambda n: x[n].to(dtype).double() if n != "gk" else x[n].double()
    st = orc.staged_forward(rd("q"), rd("k"), rd("v"), rd("a"), rd("b"), rd("gk"), R, scale,
                            x["h0"] if use_h0 else None, 64)
    g = orc.staged_backward(st, x["do"].to(dtype).double(), x["dht"] if use_dht else None)
    out = dict(o=st["o_bthv"], ht=st["ht"])
    out.update({n: g[n] for n in GRADS + (["dh0"] if use_h0 else [])})
    return out


def assert_close(got, ref, tol, label=""):
    bad = []
    for n, r in ref.items():
        e = orc.rel_err(got[n], r)
        if not e < tol:
            bad.append(f"{n}: {e:.3e}")
    assert not bad, f"{label} exceeds {tol}: " + ", ".join(bad)


@pytest.mark.parametrize("chunk", [64, 16])
def test_chunk_cfg0_fp32(dev, chunk):
    """B2 T256 H4 K=V=64 fp32 seed 0, zero initial state: o, final state and all gradients."""
    x = make_inputs(2, 256, 4, 64, 64, R, seed=0, with_dht=True)
    got = run_chunk(x, dev, 1.0, chunk, False, False, torch.float32)
    ref = oracle_chunk(x, 1.0, False, False, torch.float32)
    assert_close(got, ref, 1e-4, f"cfg0 chunk={chunk}")


def test_chunk_cfg0_against_reference_golden(dev, golden_dir):
    z = np.load(os.path.join(golden_dir, "naive_cfg0.npz"))
    x = make_inputs(2, 256, 4, 64, 64, R, seed=0, with_dht=True)
    got = run_chunk(x, dev, 1.0, 64, False, False, torch.float32)
    for n in ["o", "ht"] + GRADS:
        sub = torch.from_numpy(z["sub_" + n])
        assert orc.rel_err(got[n].reshape(-1)[::13], sub) < 1e-4, n


@pytest.mark.parametrize("chunk", [16, 32, 64])
def test_chunk_small_golden_strong_decay(dev, golden_dir, chunk):
    """Reference golden case: undivided logsigmoid decay, random h0 and dht, K=32, V=48."""
    z = np.load(os.path.join(golden_dir, "naive_small.npz"))
    x = {n[3:]: torch.from_numpy(z[n]) for n in z.files if n.startswith("in_")}
    ref = {n[4:]: torch.from_numpy(z[n]) for n in z.files if n.startswith("out_")}
    got = run_chunk(x, dev, 1.0, chunk, True, True, torch.float32)
    assert_close(got, ref, 1e-4, f"golden small chunk={chunk}")


def test_chunk_ragged_scale_h0(dev):
    """T not a multiple of the chunk, K != V, non-unit scale, initial state and dht."""
    x = make_inputs(2, 83, 3, 32, 64, R, seed=3, gk_div=4.0, h0_std=0.5, with_dht=True)
    got = run_chunk(x, dev, 0.37, 32, True, True, torch.float32)
    ref = oracle_chunk(x, 0.37, True, True, torch.float32)
    assert_close(got, ref, 1e-4, "ragged")


def test_chunk_short_sequence(dev):
    """T < 16: the effective chunk is max(next_pow2(T), 16)."""
    x = make_inputs(1, 5, 2, 16, 16, R, seed=4, gk_div=2.0, h0_std=1.0, with_dht=True)
    got = run_chunk(x, dev, 0.25, 64, True, True, torch.float32)
    ref = oracle_chunk(x, 0.25, True, True, torch.float32)
    assert_close(got, ref, 1e-4, "short")


def test_chunk_bf16(dev):
    x = make_inputs(2, 256, 2, 128, 128, R, seed=1, dtype=torch.bfloat16, with_dht=True)
    x["gk"] = x["gk"].float()
    got = run_chunk(x, dev, 128 ** -0.5, 64, False, True, torch.bfloat16)
    ref = oracle_chunk(x, 128 ** -0.5, False, True, torch.bfloat16)
    assert_close(got, ref, 2e-2, "bf16")
    assert got["o"].dtype == torch.bfloat16 and got["dq"].dtype == torch.bfloat16 and got["ht"].dtype == torch.float32


def test_chunk_recompute_equals_saved(dev, monkeypatch):
    x = make_inputs(1, 128, 2, 64, 64, R, seed=2, h0_std=0.1, with_dht=True)
    a = run_chunk(x, dev, 1.0, 64, True, True, torch.float32)
    monkeypatch.setenv("HDLA_RECOMPUTE", "1")
    b = run_chunk(x, dev, 1.0, 64, True, True, torch.float32)
    for n in a:
        assert torch.equal(a[n], b[n]), n


def test_chunk_forward_only_no_grad(dev):
    import hdla_impl_b200 as H
    x = make_inputs(1, 64, 2, 64, 64, R, seed=6)
    with torch.no_grad():
        o, ht = H.chunk_hrdplr_delta_rule(*[x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")], R,
                                          chunk_size=64)
    assert ht is None
    ref, _ = orc.recurrent_ref(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, None, None)
    assert orc.rel_err(o, ref) < 1e-4


# ---------------------------------------------------------------------------------- recurrent
def test_recurrent_cfg0_fp32(dev):
    import hdla_impl_b200 as H
    x = make_inputs(2, 256, 4, 64, 64, R, seed=0, h0_std=0.02)
    o, ht = H.fused_recurrent_dplr_delta_rule(*[x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")], R,
                                              scale=1.0, initial_state=x["h0"].to(dev), output_final_state=True)
    ro, rh = orc.recurrent_ref(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, 1.0, x["h0"])
    assert orc.rel_err(o, ro) < 1e-4 and orc.rel_err(ht, rh) < 1e-4


def test_recurrent_matches_chunk(dev):
    """The reference's test_recurrent.py: chunked and recurrent paths agree."""
    import hdla_impl_b200 as H
    x = make_inputs(2, 256, 4, 128, 64, R, seed=8, gk_div=1.0, h0_std=1.0)
    args = [x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")]
    o1, h1 = H.chunk_hrdplr_delta_rule(*args, R, scale=1.0, initial_state=x["h0"].to(dev), output_final_state=True,
                                       chunk_size=16)
    o2, h2 = H.fused_recurrent_dplr_delta_rule(*args, R, 1.0, x["h0"].to(dev), True, False, None)
    assert orc.rel_err(o1, o2) < 1e-4 and orc.rel_err(h1, h2) < 1e-4


@pytest.mark.parametrize("K,V", [(32, 48), (96, 64), (128, 128), (16, 4)])
def test_recurrent_shapes_bf16_decode(dev, K, V):
    """One token per call for several calls with a carried fp32 state (the decode loop)."""
    import hdla_impl_b200 as H
    steps, B, Hh = 6, 3, 2
    x = make_inputs(B, steps, Hh, K, V, R, seed=9, dtype=torch.bfloat16, h0_std=0.02)
    S = x["h0"].to(dev)
    outs = []
    for t in range(steps):
        sl = lambda n, r=1: x[n][:, t * r:(t + 1) * r].to(dev)
        o, S = H.fused_recurrent_dplr_delta_rule(sl("q"), sl("k"), sl("v"), sl("a", R), sl("b", R), sl("gk"), R,
                                                 initial_state=S, output_final_state=True)
        outs.append(o)
    o = torch.cat(outs, 1)
    f = lambda n: x[n].double()
    ro, rh = orc.recurrent_ref(f("q"), f("k"), f("v"), f("a"), f("b"), f("gk"), R, None, x["h0"])
    assert orc.rel_err(o, ro) < 2e-2 and orc.rel_err(S, rh) < 1e-4


@pytest.mark.parametrize("seed", range(6))
def test_recurrent_random_shapes_against_oracle(dev, seed):
    """Seeded random problems of the recurrent path: any K up to 256, V a multiple of 4 up to 256, few tokens (state
    staged in shared memory by bulk copies where it fits) or many (state in registers), forward or reverse, with or
    without an initial state, fp32 or bf16."""
    import random
    import hdla_impl_b200 as H
    rng = random.Random(2000 + seed)
    B, Hh = rng.choice([1, 2, 3]), rng.choice([1, 2])
    K, V = rng.randint(1, 256), 4 * rng.randint(1, 64)
    T = rng.choice([1, 2, 5, 8, 9, 23])
    dtype = rng.choice([torch.float32, torch.bfloat16])
    reverse, use_h0 = rng.random() < 0.4, rng.random() < 0.7
    x = make_inputs(B, T, Hh, K, V, R, seed=300 + seed, dtype=dtype, gk_div=2.0, h0_std=0.3)
    args = [x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")]
    o, ht = H.fused_recurrent_dplr_delta_rule(*args, R, 0.5, x["h0"].to(dev) if use_h0 else None, True, reverse, None)
    f = lambda n: x[n].double()
    ro, rh = orc.recurrent_ref(f("q"), f("k"), f("v"), f("a"), f("b"), f("gk"), R, 0.5, x["h0"] if use_h0 else None,
                               reverse=reverse)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    label = f"B{B} T{T} H{Hh} K{K} V{V} {dtype} reverse={reverse} h0={use_h0}"
    assert orc.rel_err(o, ro) < tol, label
    assert orc.rel_err(ht, rh) < (1e-4 if dtype == torch.float32 else 2e-2), label
    from hdla_impl_b200.recurrent import check_recurrent_status
    check_recurrent_status(dev)


def test_recurrent_inplace_state(dev):
    import hdla_impl_b200 as H
    x = make_inputs(4, 1, 2, 64, 64, R, seed=10, h0_std=0.5)
    args = [x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")]
    S = x["h0"].to(dev).clone()
    o1, h1 = H.fused_recurrent_dplr_delta_rule_fwd(*args, R, 0.125, x["h0"].to(dev), True)
    o2, h2 = H.fused_recurrent_dplr_delta_rule_fwd(*args, R, 0.125, S, True, inplace_state=True)
    assert h2.data_ptr() == S.data_ptr() and torch.equal(h1, S) and torch.equal(o1, o2)


def test_recurrent_reverse_and_varlen(dev):
    import hdla_impl_b200 as H
    x = make_inputs(1, 40, 2, 64, 32, R, seed=5, gk_div=2.0)
    args = [x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")]
    cu = torch.tensor([0, 13, 40], device=dev)
    h0 = torch.randn(2, 2, 64, 32, generator=torch.Generator().manual_seed(1))
    o, ht = H.fused_recurrent_dplr_delta_rule(*args, R, None, h0.to(dev), True, False, cu)
    ro, rh = orc.recurrent_ref(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, None, h0, cu_seqlens=[0, 13, 40])
    assert orc.rel_err(o, ro) < 1e-4 and orc.rel_err(ht, rh) < 1e-4
    o, ht = H.fused_recurrent_dplr_delta_rule(*args, R, None, None, True, True, None)
    ro, rh = orc.recurrent_ref(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, None, None, reverse=True)
    assert orc.rel_err(o, ro) < 1e-4 and orc.rel_err(ht, rh) < 1e-4


def test_recurrent_backward_raises(dev):
    import hdla_impl_b200 as H
    x = make_inputs(1, 4, 1, 16, 16, R, seed=11)
    args = [x[n].to(dev).requires_grad_(True) for n in ("q", "k", "v", "a", "b", "gk")]
    o, _ = H.fused_recurrent_dplr_delta_rule(*args, R)
    with pytest.raises(NotImplementedError):
        o.sum().backward()


def test_error_paths(dev):
    import hdla_impl_b200 as H
    x = make_inputs(1, 32, 1, 16, 16, R, seed=12)
    args = [x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")]
    with pytest.raises(RuntimeError, match="power of two"):
        H.chunk_hrdplr_delta_rule(*args, R, chunk_size=24)
    with pytest.raises(AssertionError):
        H.chunk_hrdplr_delta_rule(*args, R, head_first=True)
    with pytest.raises(ValueError):
        H.chunk_hrdplr_delta_rule(args[0], args[1], args[2], args[3][:, :-1], args[4], args[5], R)
    with pytest.raises(RuntimeError, match="CUDA"):
        H.chunk_hrdplr_delta_rule(*[x[n] for n in ("q", "k", "v", "a", "b", "gk")], R)


def test_bf16_decay_overflow_falls_back_to_fp32_pipeline(dev, monkeypatch):
    """A chunk whose total log decay exceeds what the bf16 pipeline represents must neither pass silently nor
    abort a model the reference can train: forward notices (status word 1), reruns the call on the fp32
    pipeline, and backward follows; forward + backward then match the oracle.  With HDLA_ASYNC_STATUS=1 the
    overflow is reported at the next entry instead."""
    import hdla_impl_b200 as H
    x = make_inputs(1, 128, 1, 128, 128, R, seed=13, dtype=torch.bfloat16, h0_std=0.1, with_dht=True)
    x["gk"] = torch.full_like(x["gk"].float(), -3.0)            # 64 * 3 = 192 > 150 per chunk
    # forward waits for its own status words on a device's first call and while the largest chunk decay seen there
    # is above half the limit; earlier tests of this process ran mild decays, so start from a fresh history
    H.hrdplr._status_state(dev)["decay"] = None
    with pytest.warns(RuntimeWarning, match="fp32 CUDA-core pipeline"):
        H.hrdplr._warned_fallback = False
        got = run_chunk(x, dev, 128 ** -0.5, 64, True, True, torch.bfloat16)
    assert H.hrdplr._status_state(dev)["decay"] > 150.0          # ... and from now on every call is checked
    H.check_status(dev, wait=True)
    ref = oracle_chunk(x, 128 ** -0.5, True, True, torch.bfloat16)
    assert_close(got, ref, 2e-2, "decay overflow, automatic fp32 fallback")
    # the recompute mode (inputs only are saved) has to remember the fallback too
    monkeypatch.setenv("HDLA_RECOMPUTE", "1")
    got = run_chunk(x, dev, 128 ** -0.5, 64, True, True, torch.bfloat16)
    H.check_status(dev, wait=True)
    assert_close(got, ref, 2e-2, "decay overflow, recompute mode")
    monkeypatch.delenv("HDLA_RECOMPUTE")
    # opting out of the synchronous check: reported at the next entry on that device
    monkeypatch.setenv("HDLA_ASYNC_STATUS", "1")
    args = [x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")]
    H.chunk_hrdplr_delta_rule(*args, R, chunk_size=64)
    with pytest.raises(RuntimeError, match="log decay"):
        H.check_status(dev, wait=True)
    monkeypatch.delenv("HDLA_ASYNC_STATUS")
    monkeypatch.setenv("HDLA_FORCE_SIMT", "1")
    o, ht = H.chunk_hrdplr_delta_rule(*args, R, chunk_size=64, output_final_state=True)
    H.check_status(dev, wait=True)
    f = lambda n: x[n].double()
    ro, rh = orc.recurrent_ref(f("q"), f("k"), f("v"), f("a"), f("b"), f("gk"), R, None, None)
    assert orc.rel_err(o, ro) < 2e-2 and orc.rel_err(ht, rh) < 1e-3


def test_bf16_tensor_core_path_at_reference_decay_strength(dev):
    """The reference's own tests and layer feed undivided logsigmoid decays (test_integrated.py:37-39,
    HRDPLR/hdla_custom.py:219): total log decay of a 64-chunk around 50-75, accumulator entries outside the
    masks up to e^75.  Forward + backward on the tcgen05 pipeline, initial state and final-state gradient
    included, T long enough for the two-level scan; all tensors within 2e-2 and the status words clean."""
    import ctypes as C
    import hdla_impl_b200 as H
    from hdla_impl_b200 import _lib, hrdplr
    for (B, T, Hh) in ((2, 512, 2), (1, 2048, 2)):
        x = make_inputs(B, T, Hh, 128, 128, R, seed=41, dtype=torch.bfloat16, gk_div=1.0, h0_std=0.5, with_dht=True)
        x["gk"] = x["gk"].float()
        d = hrdplr._dims(x["q"], x["v"], x["a"], x["gk"], R, 64)
        assert _lib.load().hdla_chunk_uses_tensor_cores(C.byref(d)) == 1
        got = run_chunk(x, dev, 128 ** -0.5, 64, True, True, torch.bfloat16)
        H.check_status(dev, wait=True)
        ref = oracle_chunk(x, 128 ** -0.5, True, True, torch.bfloat16)
        assert_close(got, ref, 2e-2, f"gk_div=1 B{B} T{T}")
    assert hrdplr._status_state(dev)["decay"] > 40.0         # the decay really was of the reference's strength


@pytest.mark.parametrize("B,T,H,K,V", [(2, 512, 2, 64, 64), (1, 300, 3, 128, 64), (1, 256, 2, 64, 128),
                                       (1, 200, 2, 96, 48), (1, 2100, 2, 64, 64),
                                       (2, 200, 2, 56, 40), (1, 130, 3, 120, 120), (1, 100, 2, 8, 8)])   # rows of V = 8 (mod 16)
                                                                             # elements start on odd multiples of 16 bytes
def test_bf16_head_dims_below_128_run_on_tensor_cores(dev, B, T, H, K, V):
    """The reference handles any K <= 256 and any V (HRDPLR/fwd_func.py:229-241).  Head dims below 128 (multiples
    of 8) run on the tcgen05 pipeline too, zero-padded to its 128-wide tiles: forward + backward with an initial
    state and a final-state gradient against the oracle, ragged last chunk and two-level scan included."""
    import ctypes as C
    from hdla_impl_b200 import _lib, hrdplr
    import hdla_impl_b200 as HD
    x = make_inputs(B, T, H, K, V, R, seed=51, dtype=torch.bfloat16, gk_div=4.0, h0_std=0.3, with_dht=True)
    x["gk"] = x["gk"].float()
    d = hrdplr._dims(x["q"], x["v"], x["a"], x["gk"], R, 64)
    assert _lib.load().hdla_chunk_uses_tensor_cores(C.byref(d)) == 1
    n0 = _lib.kernel_launches()
    got = run_chunk(x, dev, K ** -0.5, 64, True, True, torch.bfloat16)
    assert _lib.kernel_launches() - n0 <= 14                   # the tensor-core pipeline, not the 43-launch fp32 one
    HD.check_status(dev, wait=True)
    ref = oracle_chunk(x, K ** -0.5, True, True, torch.bfloat16)
    assert_close(got, ref, 2e-2, f"K={K} V={V}")
    # outputs must be dense [.., K] / [.., V] tensors with nothing written past their ends (NaN canaries would show
    # in the comparison above); and a forward-only call agrees bit for bit
    with torch.no_grad():
        o2, ht2 = HD.chunk_hrdplr_delta_rule(*[x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")], R,
                                             scale=K ** -0.5, initial_state=x["h0"].to(dev), output_final_state=True,
                                             chunk_size=64)
    assert torch.equal(o2, got["o"]) and torch.equal(ht2, got["ht"])


@pytest.mark.parametrize("seed", range(8))
def test_bf16_random_shapes_against_oracle(dev, seed):
    """Seeded random problems of the tensor-core pipeline (batch, ragged length, heads, head dims that are multiples
    of 8 up to 128, decay strength, with or without initial state / final-state gradient, gk in bf16 or fp32):
    forward + backward against the fp64 oracle, status words clean."""
    import random
    import hdla_impl_b200 as HD
    rng = random.Random(1000 + seed)
    B, H = rng.choice([1, 2, 3]), rng.choice([1, 2, 3])
    T = rng.randint(33, 700)
    K, V = 8 * rng.randint(1, 16), 8 * rng.randint(1, 16)
    use_h0, use_dht = rng.random() < 0.6, rng.random() < 0.6
    gk_div = rng.choice([1.0, 2.0, 8.0, 16.0])
    x = make_inputs(B, T, H, K, V, R, seed=200 + seed, dtype=torch.bfloat16, gk_div=gk_div, h0_std=0.2, with_dht=True)
    if rng.random() < 0.5:
        x["gk"] = x["gk"].float()
    scale = rng.choice([1.0, K ** -0.5])
    got = run_chunk(x, dev, scale, 64, use_h0, use_dht, torch.bfloat16)
    HD.check_status(dev, wait=True)
    ref = oracle_chunk(x, scale, use_h0, use_dht, torch.bfloat16)
    assert_close(got, ref, 2e-2, f"B{B} T{T} H{H} K{K} V{V} h0={use_h0} dht={use_dht} gk/{gk_div} {x['gk'].dtype}")


@pytest.mark.parametrize("seed", range(6))
def test_fp32_random_shapes_against_oracle(dev, seed):
    """Seeded random problems of the fp32 pipeline: any head dims (odd ones included, as the reference takes any
    K <= 256 and any V), ragged lengths, chunk 16 / 32 / 64, strong and weak decay: forward + backward, 1e-4."""
    import random
    rng = random.Random(3000 + seed)
    B, H = rng.choice([1, 2]), rng.choice([1, 2, 3])
    T = rng.randint(17, 300)
    K, V = rng.randint(1, 160), rng.randint(1, 160)
    chunk = rng.choice([16, 32, 64])
    use_h0, use_dht = rng.random() < 0.6, rng.random() < 0.6
    gk_div = rng.choice([1.0, 4.0, 16.0])
    x = make_inputs(B, T, H, K, V, R, seed=400 + seed, gk_div=gk_div, h0_std=0.2, with_dht=True)
    scale = rng.choice([1.0, K ** -0.5])
    got = run_chunk(x, dev, scale, chunk, use_h0, use_dht, torch.float32)
    ref = oracle_chunk(x, scale, use_h0, use_dht, torch.float32)
    assert_close(got, ref, 1e-4, f"B{B} T{T} H{H} K{K} V{V} chunk {chunk} h0={use_h0} dht={use_dht} gk/{gk_div}")


@pytest.mark.parametrize("seed", range(4))
def test_bf16_random_long_sequences_two_level_scan(dev, seed):
    """Seeded random long sequences with few (batch, head) pairs, where the scans run segment-parallel: random
    length (ragged), pairs, head dims, initial state and final-state gradient, against the fp64 oracle."""
    import random
    import hdla_impl_b200 as HD
    rng = random.Random(5000 + seed)
    B, H = rng.choice([(1, 1), (1, 2), (2, 1), (1, 3), (2, 2)])
    T = rng.randint(1500, 5000)
    K, V = 8 * rng.randint(4, 16), 8 * rng.randint(4, 16)
    use_h0, use_dht = rng.random() < 0.7, rng.random() < 0.7
    x = make_inputs(B, T, H, K, V, R, seed=600 + seed, dtype=torch.bfloat16, gk_div=rng.choice([4.0, 16.0]),
                    h0_std=0.2, with_dht=True)
    got = run_chunk(x, dev, K ** -0.5, 64, use_h0, use_dht, torch.bfloat16)
    HD.check_status(dev, wait=True)
    ref = oracle_chunk(x, K ** -0.5, use_h0, use_dht, torch.bfloat16)
    assert_close(got, ref, 2e-2, f"B{B} T{T} H{H} K{K} V{V} h0={use_h0} dht={use_dht}")


def _varlen_case(dev, lens, H, K, V, dtype, tol, seed):
    """Packed sequences through chunk_hrdplr_delta_rule(cu_seqlens=...) against the oracle run per sequence."""
    import hdla_impl_b200 as HD
    T = sum(lens)
    N = len(lens)
    x = make_inputs(1, T, H, K, V, R, seed=seed, dtype=dtype, gk_div=4.0)
    x["gk"] = x["gk"].float()
    g = torch.Generator().manual_seed(seed + 1)
    h0 = torch.randn(N, H, K, V, generator=g) * 0.3
    dht = torch.randn(N, H, K, V, generator=g)
    cu = [0]
    for n_ in lens:
        cu.append(cu[-1] + n_)
    names = ("q", "k", "v", "a", "b", "gk")
    lv = [x[n].to(dev).requires_grad_(True) for n in names]
    h0d = h0.to(dev).requires_grad_(True)
    o, ht = HD.chunk_hrdplr_delta_rule(*lv, R, scale=K ** -0.5, initial_state=h0d, output_final_state=True,
                                       chunk_size=64, cu_seqlens=torch.tensor(cu, device=dev))
    assert ht.shape == (N, H, K, V)
    loss = (o.float() * x["do"].to(dev).float()).sum() + (ht * dht.to(dev)).sum()
    grads = torch.autograd.grad(loss, lv + [h0d])
    HD.check_status(dev, wait=True)
    rr = lambda n: R if n in ("a", "b") else 1
    bad = []
    for s_, (lo, hi) in enumerate(zip(cu, cu[1:])):
        if hi == lo:
            assert orc.rel_err(ht[s_], h0[s_]) < 1e-6 and orc.rel_err(grads[6][s_], dht[s_]) < 1e-6
            continue
        f = lambda n: (x[n].to(dtype) if n != "gk" else x[n])[:, lo * rr(n):hi * rr(n)].double()
        st = orc.staged_forward(*[f(n) for n in names], R, K ** -0.5, h0[s_:s_ + 1], 64)
        gr = orc.staged_backward(st, x["do"].to(dtype)[:, lo:hi].double(), dht[s_:s_ + 1])
        pairs = [("o", o[:, lo:hi], st["o_bthv"]), ("ht", ht[s_:s_ + 1], st["ht"]), ("dh0", grads[6][s_:s_ + 1], gr["dh0"])]
        pairs += [(gn, t[:, lo * rr(n):hi * rr(n)], gr[gn]) for gn, t, n in zip(GRADS, grads[:6], names)]
        for name, got, ref in pairs:
            e = orc.rel_err(got, ref)
            if not e < tol:
                bad.append(f"seq {s_} {name}: {e:.3e}")
    assert not bad, "; ".join(bad)
    return o, ht


def test_chunked_varlen_packed_sequences_on_tensor_cores(dev):
    """cu_seqlens in the chunked path (the reference plumbs it into its chunk kernels, HRDPLR/fwd_triton.py:618-623,
    HRDPLR/bwd_triton.py:919-924): four packed sequences -- ragged, exactly one chunk, several chunks, a single
    token -- each with its own initial state and final-state gradient; forward and every gradient against the oracle
    run per sequence, on the tcgen05 pipeline (one launch sequence for the whole packed batch)."""
    import hdla_impl_b200 as HD
    from hdla_impl_b200 import _lib
    n0 = _lib.kernel_launches()
    o, ht = _varlen_case(dev, [200, 64, 333, 1], 2, 128, 128, torch.bfloat16, 2e-2, seed=61)
    assert _lib.kernel_launches() - n0 == 10
    # the packed result equals the sequences run one by one through the same operator
    x = make_inputs(1, 598, 2, 128, 128, R, seed=61, dtype=torch.bfloat16, gk_div=4.0)
    x["gk"] = x["gk"].float()
    h0 = torch.randn(4, 2, 128, 128, generator=torch.Generator().manual_seed(62)) * 0.3
    with torch.no_grad():
        o1, ht1 = HD.chunk_hrdplr_delta_rule(*[x[n][:, 264 * (R if n in "ab" else 1):597 * (R if n in "ab" else 1)].to(dev)
                                               for n in ("q", "k", "v", "a", "b", "gk")], R, scale=128 ** -0.5,
                                             initial_state=h0[2:3].to(dev), output_final_state=True, chunk_size=64)
    assert torch.equal(o1, o[:, 264:597]) and torch.equal(ht1, ht[2:3])
    # head dims below 128 and an empty sequence in the middle
    _varlen_case(dev, [70, 0, 130], 3, 64, 64, torch.bfloat16, 2e-2, seed=63)


@pytest.mark.parametrize("seed", range(4))
def test_chunked_varlen_random_batches(dev, seed):
    """Seeded random packed batches on the tensor-core pipeline: two to six sequences of 0 .. 300 tokens (empty ones,
    single tokens and exact chunk multiples included), random heads and head dims."""
    import random
    rng = random.Random(4000 + seed)
    lens = [rng.choice([0, 1, 63, 64, 65, 128, rng.randint(2, 300)]) for _ in range(rng.randint(2, 6))]
    if sum(lens) <= 32:
        lens.append(100)
    H, K, V = rng.choice([1, 2, 3]), 8 * rng.randint(1, 16), 8 * rng.randint(1, 16)
    _varlen_case(dev, lens, H, K, V, torch.bfloat16, 2e-2, seed=500 + seed)


def test_chunked_varlen_falls_back_to_per_sequence_calls(dev):
    """Problems outside the tensor-core pipeline (here fp32) take cu_seqlens too: sequence by sequence."""
    _varlen_case(dev, [50, 64, 17], 2, 32, 48, torch.float32, 1e-4, seed=65)
    with pytest.raises(ValueError, match="batch size"):
        import hdla_impl_b200 as HD
        x = make_inputs(2, 64, 1, 32, 32, R, seed=1)
        HD.chunk_hrdplr_delta_rule(*[x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")], R, cu_seqlens=[0, 64])


def test_non_contiguous_inputs_and_autocast(dev):
    """The entry point makes its tensor arguments contiguous and is autocast-aware like the reference's
    decorators (HRDPLR/utils.py:7-25, HRDPLR/hrdplr.py:104-105,148-149)."""
    import hdla_impl_b200 as H
    x = make_inputs(2, 128, 2, 128, 128, R, seed=43, dtype=torch.bfloat16)
    x["gk"] = x["gk"].float()
    names = ("q", "k", "v", "a", "b", "gk")
    ref = oracle_chunk(x, 128 ** -0.5, False, False, torch.bfloat16)
    # q and v as transposed views of [B, H, T, K] storage; k with a strided last-but-one dimension
    lv = []
    for n in names:
        t = x[n].to(dev)
        if n in ("q", "v"):
            t = t.permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3)
            assert not t.is_contiguous()
        lv.append(t.requires_grad_(True))
    o, _ = H.chunk_hrdplr_delta_rule(*lv, R, chunk_size=64)
    grads = torch.autograd.grad(o, lv, x["do"].to(dev).permute(0, 2, 1, 3).contiguous().permute(0, 2, 1, 3))
    got = dict(o=o, **dict(zip(GRADS, grads)))
    assert_close(got, {n: ref[n] for n in got}, 2e-2, "non-contiguous")
    # fp32 tensors inside a bf16 autocast region: like the reference's decorators (custom_fwd without cast_inputs)
    # the operator keeps the dtype it is given, so this runs the fp32 pipeline and returns fp32
    lv32 = [x[n].float().to(dev).requires_grad_(True) for n in names]
    with torch.autocast("cuda", dtype=torch.bfloat16):
        o32, _ = H.chunk_hrdplr_delta_rule(*lv32, R, chunk_size=64)
        g32 = torch.autograd.grad(o32, lv32, x["do"].float().to(dev))
    assert o32.dtype == torch.float32 and all(g.dtype == torch.float32 for g in g32)
    got = dict(o=o32, **dict(zip(GRADS, g32)))
    assert_close(got, {n: ref[n] for n in got}, 1e-4, "autocast region, fp32 inputs")
    H.check_status(dev, wait=True)


def test_device_wait_timeout_is_reported_and_context_survives(dev):
    """Failure detection without a fault: a kernel whose wait can never succeed gives up after its time budget,
    records the wait code in status word 0 and returns; the host turns the word into an exception; the next
    ordinary call on the same context succeeds."""
    import ctypes as C
    import hdla_impl_b200 as H
    from hdla_impl_b200 import _lib, hrdplr
    lib = _lib.load()
    ws = torch.zeros(256, dtype=torch.uint8, device=dev)
    rc = lib.hdla_debug_wait_timeout(_lib.ptr(ws), C.c_uint64(2_000_000), _lib.stream_ptr(dev))     # 2 ms budget
    _lib.check(rc, "hdla_debug_wait_timeout")
    hrdplr._post_status(ws, dev)
    with pytest.raises(RuntimeError, match="device-side wait ran out"):
        H.check_status(dev, wait=True)
    assert ws[:4].view(torch.int32).item() == 99
    x = make_inputs(1, 128, 2, 128, 128, R, seed=44, dtype=torch.bfloat16)
    x["gk"] = x["gk"].float()
    got = run_chunk(x, dev, 128 ** -0.5, 64, False, False, torch.bfloat16)
    H.check_status(dev, wait=True)
    ref = oracle_chunk(x, 128 ** -0.5, False, False, torch.bfloat16)
    assert_close(got, ref, 2e-2, "call after a reported timeout")


def test_prefill_then_decode_state_handoff(dev):
    """final_state of the chunked call seeds the recurrent calls (the reference layer's cache path,
    HRDPLR/hdla_custom.py:295-337): prefill T0 tokens chunked, then decode token by token."""
    import hdla_impl_b200 as H
    T0, T1 = 192, 5
    x = make_inputs(2, T0 + T1, 2, 128, 128, R, seed=14, dtype=torch.bfloat16)
    names = ("q", "k", "v", "a", "b", "gk")
    rr = lambda n: R if n in ("a", "b") else 1
    pre = [x[n][:, :T0 * rr(n)].to(dev) for n in names]
    o0, S = H.chunk_hrdplr_delta_rule(*pre, R, output_final_state=True, chunk_size=64)
    outs = [o0]
    for t in range(T0, T0 + T1):
        cur = [x[n][:, t * rr(n):(t + 1) * rr(n)].to(dev) for n in names]
        o, S = H.fused_recurrent_dplr_delta_rule(*cur, R, initial_state=S, output_final_state=True)
        outs.append(o)
    o = torch.cat(outs, 1)
    f = lambda n: x[n].double()
    ro, rh = orc.recurrent_ref(f("q"), f("k"), f("v"), f("a"), f("b"), f("gk"), R, None, None)
    assert orc.rel_err(o, ro) < 2e-2 and orc.rel_err(S, rh) < 2e-2


def test_host_pipeline_matches_device_call(dev):
    """chunk_fwd_bwd_from_host (pinned host tensors, sliced and pipelined over streams) equals one device call."""
    import hdla_impl_b200 as H
    from hdla_impl_b200.host import chunk_fwd_bwd_from_host
    x = make_inputs(3, 128, 2, 128, 128, R, seed=15, dtype=torch.bfloat16)
    names = ("q", "k", "v", "a", "b", "gk")
    host = {n: x[n].pin_memory() for n in names + ("do",)}
    out = chunk_fwd_bwd_from_host(host, None, R, dev, chunk_size=64, slice_batch=1)
    lv = [x[n].to(dev).requires_grad_(True) for n in names]
    o, _ = H.chunk_hrdplr_delta_rule(*lv, R, chunk_size=64)
    g = torch.autograd.grad(o, lv, x["do"].to(dev))
    for n, t in zip(("o", "dq", "dk", "dv", "da", "db", "dgk"), (o,) + tuple(g)):
        assert torch.equal(out[n], t.detach().cpu()), n


def test_host_pipeline_streams_across_calls(dev):
    """With sync=False successive calls only enqueue; after one synchronisation every call's results are there."""
    from hdla_impl_b200.host import chunk_fwd_bwd_from_host
    names = ("q", "k", "v", "a", "b", "gk")
    hosts, outs, refs = [], [], []
    for seed in (21, 22, 23):
        x = make_inputs(2, 128, 2, 128, 128, R, seed=seed, dtype=torch.bfloat16)
        hosts.append({n: x[n].pin_memory() for n in names + ("do",)})
    for h in hosts:
        refs.append({k: v.clone() for k, v in chunk_fwd_bwd_from_host(h, None, R, dev, chunk_size=64).items()})
    for h in hosts:                                   # enqueue all three, synchronise once
        outs.append(chunk_fwd_bwd_from_host(h, None, R, dev, chunk_size=64, sync=False))
    torch.cuda.synchronize(dev)
    for o, r in zip(outs, refs):
        for n in r:
            assert torch.equal(o[n], r[n]), n


@pytest.mark.parametrize("B,T,H", [(1, 200, 3), (2, 1000, 5), (3, 2048, 7)])
def test_repeated_calls_are_bit_identical(dev, B, T, H):
    """No kernel accumulates with atomics, so repeated calls on the same inputs must agree bit for bit: a
    difference would mean a race between the loads, products and epilogues of the pipelined kernels (tile counts
    below, above and not a multiple of the persistent grids; ragged last chunk; h0 and dht given)."""
    import hdla_impl_b200 as H_
    x = make_inputs(B, T, H, 128, 128, R, seed=B * 100 + H, dtype=torch.bfloat16)
    names = ("q", "k", "v", "a", "b", "gk")
    lv = [x[n].to(dev).requires_grad_(True) for n in names]
    do = x["do"].to(dev)
    h0 = (torch.randn(B, H, 128, 128, generator=torch.Generator().manual_seed(5)) * 0.02).to(dev)
    ref = None
    for _ in range(4):
        o, ht = H_.chunk_hrdplr_delta_rule(*lv, R, chunk_size=64, initial_state=h0, output_final_state=True)
        g = torch.autograd.grad([o, ht], lv, [do, torch.full_like(ht, 0.01)])
        cur = [o.detach().clone(), ht.detach().clone()] + [t.clone() for t in g]
        if ref is None:
            ref = cur
        else:
            for i, (a_, b_) in enumerate(zip(cur, ref)):
                assert torch.equal(a_, b_), f"tensor {i} differs between repeated calls"
    H_.check_status()


def _param_ab_torch(beta, k, log_f):
    """The oracle's restatement of the reference's parameterize_a_b (HRDPLR/hdla_custom.py:19-43), pinned by
    tests/golden/param_ab_small.npz (tests/test_oracle.py)."""
    return orc.param_ab_ref(beta, k, log_f)


def _layer_inputs(B, T, H, K, V, seed, gk_div):
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s_: torch.randn(*s_, generator=g)
    x = dict(q=torch.nn.functional.normalize(rn(B, T, H, K), dim=-1), k=torch.nn.functional.normalize(rn(B, T, H, K), dim=-1),
             v=rn(B, T, H, V), beta=2 * torch.sigmoid(rn(B, T, H, 1)),
             log_f=torch.nn.functional.logsigmoid(rn(B, T, H, K)) / gk_div, do=rn(B, T, H, V),
             h0=0.2 * rn(B, H, K, V), dht=rn(B, H, K, V))
    return x


@pytest.mark.parametrize("B,T,H,K,V,fdt,gk_div,norm_k", [(2, 300, 2, 128, 128, torch.bfloat16, 16.0, False),
                                                         (1, 640, 3, 128, 128, torch.float32, 1.0, False),
                                                         (2, 200, 2, 64, 32, torch.bfloat16, 4.0, False),
                                                         (2, 300, 2, 128, 128, torch.bfloat16, 8.0, True),
                                                         (1, 200, 2, 96, 64, torch.float32, 4.0, True)])
def test_chunk_hdla_parametrisation_inside_the_operator(dev, B, T, H, K, V, fdt, gk_div, norm_k):
    """`chunk_hdla_delta_rule(q, k, v, beta, log_f)` -- a and b formed inside the chunk-preparation kernel, their
    backward folded into dk, dlog_f, dbeta by the library -- against the fp64 oracle fed with the a, b of the
    reference's parameterize_a_b (HRDPLR/hdla_custom.py:19-43, :290-309), and against the two-call route on the GPU.
    Ragged tails, initial state, dht, log_f in bf16 and fp32, head dims below 128, the layer's undivided decay."""
    from hdla_impl_b200.layer_ops import chunk_hdla_delta_rule, parameterize_a_b
    import hdla_impl_b200 as Hm
    from hdla_impl_b200 import _lib
    x = _layer_inputs(B, T, H, K, V, seed=31, gk_div=gk_div)
    if norm_k:                       # the layer's l2_norm of k inside the operator too: feed rows of uneven length
        x["k"] = x["k"] * (0.5 + 3 * torch.rand(B, T, H, 1, generator=torch.Generator().manual_seed(5)))
    bf = torch.bfloat16
    dts = dict(q=bf, k=bf, v=bf, beta=bf, log_f=fdt)
    names = ["q", "k", "v", "beta", "log_f"]
    # oracle in fp64 on the values the device sees
    rl = {n: x[n].to(dts[n]).double().requires_grad_(True) for n in names}
    h0r = x["h0"].double().requires_grad_(True)
    rk = rl["k"] / torch.sqrt((rl["k"] * rl["k"]).sum(-1, keepdim=True) + 1e-5) if norm_k else rl["k"]
    ra, rb = _param_ab_torch(rl["beta"], rk, rl["log_f"])
    ro, rht = orc.chunked_ref(rl["q"], rk, rl["v"], ra, rb, rl["log_f"], 2, 1.0, h0r, True, 64)
    rg = torch.autograd.grad((ro * x["do"].to(bf).double()).sum() + (rht * x["dht"].double()).sum(),
                             [rl[n] for n in names] + [h0r])
    ref = dict(o=ro, ht=rht, **{"d" + n: g_ for n, g_ in zip(names + ["h0"], rg)})

    def run(fn):
        lv = {n: x[n].to(dts[n]).to(dev).requires_grad_(True) for n in names}
        h0 = x["h0"].to(dev).requires_grad_(True)
        o, ht = fn(lv, h0)
        gr = torch.autograd.grad((o.float() * x["do"].to(bf).to(dev).float()).sum() + (ht * x["dht"].to(dev)).sum(),
                                 [lv[n] for n in names] + [h0])
        return dict(o=o, ht=ht, **{"d" + n: g_ for n, g_ in zip(names + ["h0"], gr)})

    n0 = _lib.kernel_launches()
    got = run(lambda lv, h0: chunk_hdla_delta_rule(lv["q"], lv["k"], lv["v"], lv["beta"], lv["log_f"], scale=1.0,
                                                   initial_state=h0, output_final_state=True, normalize_k=norm_k))
    launches = _lib.kernel_launches() - n0
    assert got["dbeta"].shape == x["beta"].shape and got["dlog_f"].dtype == fdt
    assert_close(got, ref, 2e-2, "in-operator parametrisation")
    if T // 64 < 8:                  # one-level scans: the ten operator kernels and the parametrisation's backward
        assert launches == 11, launches

    def two_calls(lv, h0):
        a, b = parameterize_a_b(lv["beta"], lv["k"], lv["log_f"])
        return Hm.chunk_hrdplr_delta_rule(lv["q"], lv["k"], lv["v"], a, b, lv["log_f"], 2, scale=1.0,
                                          initial_state=h0, output_final_state=True, chunk_size=64)
    if fdt == bf and not norm_k:
        assert_close(run(two_calls), ref, 2e-2, "two-call route")
    Hm.check_status(dev, wait=True)


def test_chunk_hdla_packed_sequences_recompute_and_forward_only(dev, monkeypatch):
    """The one-call layer operator on a packed variable-length batch equals its per-sequence calls; backward that
    recomputes the forward (HDLA_RECOMPUTE=1) is bit-identical to backward on the saved workspace; a no-grad
    forward (forward-only workspace) returns the same output."""
    from hdla_impl_b200.layer_ops import chunk_hdla_delta_rule
    H, K, V = 2, 128, 128
    offs = [0, 200, 264, 598]
    x = _layer_inputs(1, offs[-1], H, K, V, seed=33, gk_div=8.0)
    bf = torch.bfloat16
    names = ["q", "k", "v", "beta", "log_f"]
    h0 = 0.2 * torch.randn(len(offs) - 1, H, K, V, generator=torch.Generator().manual_seed(1))

    def run(cu, lo=0, hi=offs[-1], states=slice(None)):
        lv = [x[n][:, lo:hi].to(bf).to(dev).requires_grad_(True) for n in names]
        o, ht = chunk_hdla_delta_rule(*lv, scale=1.0, initial_state=h0[states].to(dev), output_final_state=True,
                                      cu_seqlens=cu)
        gr = torch.autograd.grad((o.float() * x["do"][:, lo:hi].to(dev)).sum() + ht.sum(), lv)
        return [o, ht] + list(gr)

    packed = run(offs)
    monkeypatch.setenv("HDLA_RECOMPUTE", "1")
    again = run(offs)
    monkeypatch.delenv("HDLA_RECOMPUTE")
    for a_, b_ in zip(packed, again):
        assert torch.equal(a_, b_)
    parts = [run(None, lo, hi, slice(i, i + 1)) for i, (lo, hi) in enumerate(zip(offs, offs[1:]))]
    for j in range(len(packed)):
        whole = torch.cat([p_[j] for p_ in parts], 0 if j == 1 else 1)
        assert orc.rel_err(packed[j], whole) < 5e-3, j
    with torch.no_grad():
        lv = [x[n].to(bf).to(dev) for n in names]
        o, ht = chunk_hdla_delta_rule(*lv, scale=1.0, initial_state=h0.to(dev), output_final_state=True, cu_seqlens=offs)
        assert torch.equal(o, packed[0]) and torch.equal(ht, packed[1])
        # a constant beta (the layer without a beta projection uses 2) is the same as a tensor filled with it
        o2, _ = chunk_hdla_delta_rule(lv[0], lv[1], lv[2], 2, lv[4], scale=1.0, cu_seqlens=offs)
        o3, _ = chunk_hdla_delta_rule(lv[0], lv[1], lv[2], torch.full_like(lv[3], 2.0), lv[4], scale=1.0, cu_seqlens=offs)
        assert torch.equal(o2, o3)


@pytest.mark.parametrize("K", [96, 128, 200, 100])   # one piece per lane, full rows, two pieces, scalar kernels
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_parameterize_a_b_forward_backward(dev, dtype, tol, K):
    from hdla_impl_b200.layer_ops import parameterize_a_b
    g = torch.Generator().manual_seed(3)
    B, T, H = 2, 33, 3
    k = torch.nn.functional.normalize(torch.randn(B, T, H, K, generator=g), dim=-1)
    beta = 2 * torch.sigmoid(torch.randn(B, T, H, 1, generator=g))
    log_f = torch.nn.functional.logsigmoid(torch.randn(B, T, H, K, generator=g))
    ga, gb = torch.randn(B, 2 * T, H, K, generator=g), torch.randn(B, 2 * T, H, K, generator=g)
    rd = lambda t: t.to(dtype).double().requires_grad_(True)
    rb, rk, rf = rd(beta), rd(k), rd(log_f)
    ra, rbb = _param_ab_torch(rb, rk, rf)
    rg = torch.autograd.grad((ra * ga.to(dtype).double()).sum() + (rbb * gb.to(dtype).double()).sum(), [rb, rk, rf])
    xb, xk, xf = (t.to(dtype).to(dev).requires_grad_(True) for t in (beta, k, log_f))
    a, b = parameterize_a_b(xb, xk, xf)
    gg = torch.autograd.grad((a.float() * ga.to(dtype).to(dev).float()).sum() + (b.float() * gb.to(dtype).to(dev).float()).sum(),
                             [xb, xk, xf])
    assert orc.rel_err(a, ra) < tol and orc.rel_err(b, rbb) < tol
    for got, ref, n in zip(gg, rg, ("dbeta", "dk", "dlog_f")):
        assert orc.rel_err(got, ref) < tol, n


def test_parameterize_a_b_against_reference_golden(dev, golden_dir):
    """The CUDA kernel against a and b computed by the reference's own function (read out of its frame by
    tests/golden/make_param_ab_golden.py)."""
    from hdla_impl_b200.layer_ops import parameterize_a_b
    z = np.load(os.path.join(golden_dir, "param_ab_small.npz"))
    beta, k, log_f = (torch.from_numpy(z[n]).float().to(dev) for n in ("beta", "k", "log_f"))
    a, b = parameterize_a_b(beta, k, log_f)
    ra, rb = orc.param_ab_ref(beta.double().cpu(), k.double().cpu(), log_f.double().cpu())   # on the fp32-rounded inputs
    assert orc.rel_err(a, ra) < 1e-6 and orc.rel_err(b, rb) < 1e-6
    assert orc.rel_err(a, torch.from_numpy(z["a"])) < 1e-5 and orc.rel_err(b, torch.from_numpy(z["b"])) < 1e-5


def test_rms_norm_fused_gate_against_reference_golden(dev, golden_dir):
    """The CUDA kernels against o, dx, dgate, dweight computed by the reference's own normalize_torch
    (tests/golden/make_norm_gate_golden.py)."""
    from hdla_impl_b200.layer_ops import rms_norm_fused_gate
    z = np.load(os.path.join(golden_dir, "norm_gate_small.npz"))
    x, gate, w = (torch.from_numpy(z[n]).to(dev).requires_grad_(True) for n in ("x", "gate", "weight"))
    o = rms_norm_fused_gate(x, gate, w, float(z["eps"]))
    grads = torch.autograd.grad((o * torch.from_numpy(z["d_o"]).to(dev)).sum(), [x, gate, w])
    assert orc.rel_err(o, torch.from_numpy(z["o"])) < 1e-5
    for got, n in zip(grads, ("dx", "dgate", "dweight")):
        assert orc.rel_err(got, torch.from_numpy(z[n])) < 1e-5, n


def test_bf16_recompute_and_forward_only(dev, monkeypatch):
    """Tensor-core path: backward that recomputes the forward (HDLA_RECOMPUTE=1, the reference's behaviour) gives
    the same gradients as backward on the saved workspace; a no-grad forward uses the forward-only workspace."""
    import hdla_impl_b200 as H
    x = make_inputs(1, 256, 2, 128, 128, R, seed=16, dtype=torch.bfloat16, h0_std=0.1, with_dht=True)
    a = run_chunk(x, dev, 0.1, 64, True, True, torch.bfloat16)
    monkeypatch.setenv("HDLA_RECOMPUTE", "1")
    b = run_chunk(x, dev, 0.1, 64, True, True, torch.bfloat16)
    for n in a:
        assert torch.equal(a[n], b[n]), n
    with torch.no_grad():
        o, ht = H.chunk_hrdplr_delta_rule(*[x[n].to(dev) for n in ("q", "k", "v", "a", "b", "gk")], R, scale=0.1,
                                          initial_state=x["h0"].to(dev), output_final_state=True, chunk_size=64)
    assert torch.equal(o, a["o"]) and torch.equal(ht, a["ht"])


@pytest.mark.parametrize("rows,D", [(37, 2048), (700, 64), (5, 4096), (3, 8192), (9, 1000)])
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
def test_rms_norm_fused_gate_forward_backward(dev, dtype, tol, rows, D):
    """Against the arithmetic of the reference's normalize_torch (c = sqrt(D), no mean, sigmoid gate applied before).
    3 x 700 rows is more than the grid holds, so every CTA walks over several rows and sums its share of dweight."""
    from hdla_impl_b200.layer_ops import rms_norm_fused_gate
    g = torch.Generator().manual_seed(5)
    eps = 1e-5
    x, gate = torch.randn(3, rows, D, generator=g), torch.randn(3, rows, D, generator=g)
    w, go = 1 + 0.1 * torch.randn(D, generator=g), torch.randn(3, rows, D, generator=g)
    rd = lambda t: t.to(dtype).double().requires_grad_(True)
    rx, rg, rw = rd(x), rd(gate), rd(w)
    ro = orc.norm_gate_ref(rx, rg, rw, eps)
    rgrads = torch.autograd.grad((ro * go.to(dtype).double()).sum(), [rx, rg, rw])
    dx, dg, dw = (t.to(dtype).to(dev).requires_grad_(True) for t in (x, gate, w))
    o = rms_norm_fused_gate(dx, dg, dw, eps)
    grads = torch.autograd.grad((o.float() * go.to(dtype).to(dev).float()).sum(), [dx, dg, dw])
    assert orc.rel_err(o, ro) < tol
    for got, ref, n in zip(grads, rgrads, ("dx", "dgate", "dweight")):
        assert orc.rel_err(got, ref) < tol, n


def test_bf16_requested_chunk_16_runs_on_tensor_cores(dev, monkeypatch):
    """The reference layer passes chunk_size=16; the result is chunk-size independent, so supported bf16
    problems still take the tensor-core pipeline (10 launches for forward+backward, 7 with the one-kernel chunk
    preparation, not the 43 of the fp32 one)."""
    import hdla_impl_b200 as H
    from hdla_impl_b200 import _lib
    x = make_inputs(1, 256, 2, 128, 128, R, seed=17, dtype=torch.bfloat16, with_dht=True)
    n0 = _lib.kernel_launches()
    a = run_chunk(x, dev, 1.0, 16, False, True, torch.bfloat16)
    assert _lib.kernel_launches() - n0 == 10
    monkeypatch.setenv("HDLA_FUSED_PREP", "1")
    n0 = _lib.kernel_launches()
    f = run_chunk(x, dev, 1.0, 16, False, True, torch.bfloat16)
    assert _lib.kernel_launches() - n0 == 7
    monkeypatch.delenv("HDLA_FUSED_PREP")
    b = run_chunk(x, dev, 1.0, 64, False, True, torch.bfloat16)
    for n in a:
        assert torch.equal(a[n], b[n]), n
    monkeypatch.setenv("HDLA_HONOR_CHUNK", "1")
    c = run_chunk(x, dev, 1.0, 16, False, True, torch.bfloat16)      # fp32 pipeline at chunk 16
    ref = oracle_chunk(x, 1.0, False, True, torch.bfloat16)
    assert_close(c, ref, 2e-2, "chunk 16 honoured")
    assert_close(a, ref, 2e-2, "chunk 16 requested")
    assert_close(f, ref, 2e-2, "chunk 16 requested, one-kernel preparation")


@pytest.mark.parametrize("T", [2000, 2100])      # 32 chunks in 4 segments; 33 chunks in 7 segments of 5
def test_bf16_two_level_scan_long_sequence(dev, T):
    """Few (batch, head) pairs and many chunks: the scan runs segment-parallel (transition + state-from-zero per
    segment, composed, then the real scan), forward and reverse.  T = 2000 -> 32 chunks in 4 segments, ragged tail,
    initial state and dht."""
    x = make_inputs(1, T, 2, 128, 128, R, seed=18, dtype=torch.bfloat16, h0_std=0.2, with_dht=True)
    x["gk"] = x["gk"].float()
    got = run_chunk(x, dev, 128 ** -0.5, 64, True, True, torch.bfloat16)
    ref = oracle_chunk(x, 128 ** -0.5, True, True, torch.bfloat16)
    assert_close(got, ref, 2e-2, "two-level scan")
