"""CPU: pin the oracle restatements to golden vectors produced by the reference's naive.py."""
import os

import numpy as np
import pytest
import torch

from oracle import hdla_oracle as orc
from hdla_impl_b200.synthetic import make_inputs

R = 2
GRADS = ["dq", "dk", "dv", "da", "db", "dgk", "dh0"]


def _small(golden_dir):
    z = np.load(os.path.join(golden_dir, "naive_small.npz"))
    x = {n[3:]: torch.from_numpy(z[n]) for n in z.files if n.startswith("in_")}
    ref = {n[4:]: torch.from_numpy(z[n]) for n in z.files if n.startswith("out_")}
    return x, ref


def test_recurrence_matches_reference_naive(golden_dir):
    x, ref = _small(golden_dir)
    o, ht = orc.recurrent_ref(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, 1.0, x["h0"])
    assert orc.rel_err(o, ref["o"]) < 1e-12
    assert orc.rel_err(ht, ref["ht"]) < 1e-12


@pytest.mark.parametrize("chunk", [16, 64])
def test_chunked_autograd_matches_reference_naive(golden_dir, chunk):
    x, ref = _small(golden_dir)
    fn = lambda q, k, v, a, b, gk, h0: orc.chunked_ref(q, k, v, a, b, gk, R, 1.0, h0, True, chunk)
    o, ht, g = orc.autograd_ref(fn, x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], x["h0"], x["do"], x["dht"])
    assert orc.rel_err(o, ref["o"]) < 1e-11
    assert orc.rel_err(ht, ref["ht"]) < 1e-11
    for n in GRADS:
        assert orc.rel_err(g[n], ref[n]) < 1e-10, n


@pytest.mark.parametrize("chunk", [16, 64])
def test_staged_backward_matches_reference_naive(golden_dir, chunk):
    x, ref = _small(golden_dir)
    st = orc.staged_forward(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, 1.0, x["h0"], chunk)
    assert orc.rel_err(st["o_bthv"], ref["o"]) < 1e-11
    assert orc.rel_err(st["ht"], ref["ht"]) < 1e-11
    g = orc.staged_backward(st, x["do"], x["dht"])
    for n in GRADS:
        assert orc.rel_err(g[n], ref[n]) < 1e-10, n


def test_recurrence_autograd_matches_reference_naive(golden_dir):
    x, ref = _small(golden_dir)
    fn = lambda q, k, v, a, b, gk, h0: orc.recurrent_ref(q, k, v, a, b, gk, R, 1.0, h0)
    o, ht, g = orc.autograd_ref(fn, x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], x["h0"], x["do"], x["dht"])
    for n in GRADS:
        assert orc.rel_err(g[n], ref[n]) < 1e-10, n


def test_cfg0_matches_reference_naive(golden_dir):
    """CPU configuration B2 T256 H4 K=V=64 seed 0 against the subsampled reference output."""
    z = np.load(os.path.join(golden_dir, "naive_cfg0.npz"))
    x = make_inputs(2, 256, 4, 64, 64, R, seed=0, gk_div=16.0, with_dht=True)
    for n in ("q", "k", "v", "a", "b", "gk", "do"):
        s = z["insum_" + n]
        assert abs(x[n].double().sum().item() - s[0]) <= 1e-6 * max(1.0, s[1]), f"input generator differs: {n}"
    st = orc.staged_forward(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, 1.0, None, 64)
    g = orc.staged_backward(st, x["do"], None)
    got = dict(o=st["o_bthv"], ht=st["ht"], **{n: g[n] for n in GRADS})
    for n, t in got.items():
        sub = torch.from_numpy(z["sub_" + n])
        assert orc.rel_err(t.reshape(-1)[::13], sub) < 1e-10, n
        assert abs(t.sum().item() - z["sum_" + n][0]) < 1e-8 * max(1.0, z["sum_" + n][1]), n


def test_scale_and_partial_chunk_consistency():
    """scale is applied to q; a ragged last chunk equals the recurrence."""
    x = make_inputs(2, 83, 2, 16, 24, R, seed=3, gk_div=4.0, h0_std=0.5, with_dht=True)
    fn_c = lambda q, k, v, a, b, gk, h0: orc.chunked_ref(q, k, v, a, b, gk, R, 0.37, h0, True, 32)
    fn_r = lambda q, k, v, a, b, gk, h0: orc.recurrent_ref(q, k, v, a, b, gk, R, 0.37, h0)
    args = [x[n] for n in ("q", "k", "v", "a", "b", "gk", "h0", "do", "dht")]
    o1, h1, g1 = orc.autograd_ref(fn_c, *args)
    o2, h2, g2 = orc.autograd_ref(fn_r, *args)
    assert orc.rel_err(o1, o2) < 1e-11 and orc.rel_err(h1, h2) < 1e-11
    for n in GRADS:
        assert orc.rel_err(g1[n], g2[n]) < 1e-10, n
    st = orc.staged_forward(*args[:6], R, 0.37, x["h0"], 32)
    g3 = orc.staged_backward(st, x["do"], x["dht"])
    for n in GRADS:
        assert orc.rel_err(g3[n], g2[n]) < 1e-10, n


def test_reverse_and_varlen_recurrence():
    x = make_inputs(1, 40, 2, 16, 16, R, seed=5, gk_div=2.0)
    cu = [0, 13, 40]
    h0 = torch.randn(2, 2, 16, 16, generator=torch.Generator().manual_seed(1))
    o, ht = orc.recurrent_ref(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, None, h0, cu_seqlens=cu)
    for i in range(2):
        s, e = cu[i], cu[i + 1]
        oi, hi = orc.recurrent_ref(x["q"][:, s:e], x["k"][:, s:e], x["v"][:, s:e], x["a"][:, 2 * s:2 * e],
                                   x["b"][:, 2 * s:2 * e], x["gk"][:, s:e], R, None, h0[i:i + 1])
        assert orc.rel_err(o[:, s:e], oi) < 1e-13 and orc.rel_err(ht[i:i + 1], hi) < 1e-13
    # reverse == forward on the time-flipped sequence
    flip2 = lambda t: t.view(1, 40, 2, 2, 16).flip(1).reshape(1, 80, 2, 16)
    orv, hrv = orc.recurrent_ref(x["q"], x["k"], x["v"], x["a"], x["b"], x["gk"], R, None, None, reverse=True)
    of, hf = orc.recurrent_ref(x["q"].flip(1), x["k"].flip(1), x["v"].flip(1), flip2(x["a"]), flip2(x["b"]),
                               x["gk"].flip(1), R, None, None)
    assert orc.rel_err(orv, of.flip(1)) < 1e-13 and orc.rel_err(hrv, hf) < 1e-13


def test_installed_reference_matches_oracle():
    """Where oracle/install_ref.py has placed the reference's own naive.py, it and the restatement agree on
    forward and autograd gradients (fp64, seeded inputs); skipped where the reference is not installed."""
    import pytest
    from oracle import ref_naive
    if not ref_naive.available():
        pytest.skip("oracle/_ref/naive.py is not installed")
    from hdla_impl_b200.synthetic import make_inputs
    x = make_inputs(1, 128, 2, 32, 32, 2, seed=11, gk_div=2.0)
    o, ht, grads = ref_naive.fwd_bwd(x, 2, 32, dtype=torch.float64)
    f = lambda n: x[n].double()
    st = orc.staged_forward(f("q"), f("k"), f("v"), f("a"), f("b"), f("gk"), 2, 1.0, None, 32)
    g = orc.staged_backward(st, f("do"), None)
    assert orc.rel_err(o, st["o_bthv"]) < 1e-10 and orc.rel_err(ht, st["ht"]) < 1e-10
    for t, n in zip(grads, ("dq", "dk", "dv", "da", "db", "dgk")):
        assert orc.rel_err(t, g[n]) < 1e-10, n


def test_oracle_scan_stage_matches_the_reference_scan_function():
    """The state-scan stage of the staged oracle (state entering every chunk, v2, final state) against the
    reference's own ``fwd_h_naive`` (HRDPLR/naive.py:11-73) fed with the oracle's stage operands; skipped where the
    reference is not installed."""
    import pytest
    from oracle import ref_naive
    if not ref_naive.available():
        pytest.skip("oracle/_ref/naive.py is not installed")
    from hdla_impl_b200.synthetic import make_inputs
    B, T, H, K, V, R, C = 2, 64, 2, 16, 24, 2, 16
    x = make_inputs(B, T, H, K, V, R, seed=13, gk_div=2.0, h0_std=0.5)
    f = lambda n: x[n].double()
    st = orc.staged_forward(f("q"), f("k"), f("v"), f("a"), f("b"), f("gk"), R, 1.0, x["h0"], C)
    # chunk-major [B,H,NT,rows,D] -> the reference's [B, NT*rows, H, D]
    flat = lambda t: t.permute(0, 2, 3, 1, 4).reshape(B, -1, H, t.shape[-1])
    h_ref, ht_ref, v_new_ref = ref_naive.load().fwd_h_naive(flat(st["kg"]), f("v"), flat(st["bg"]), flat(st["w"]),
                                                            flat(st["u"]), flat(st["gi"]), x["h0"].double(), C, R)
    assert orc.rel_err(st["h"].permute(0, 2, 1, 3, 4), h_ref) < 1e-12          # [B,H,NT,K,V] vs [B,NT,H,K,V]
    assert orc.rel_err(flat(st["v2"]), v_new_ref) < 1e-12
    assert orc.rel_err(st["ht"], ht_ref) < 1e-12


def test_param_ab_restatement_matches_the_reference_function(golden_dir):
    """``param_ab_ref`` against a and b computed by the reference's own ``parameterize_a_b`` (the function returns
    nothing; the generator read them out of its frame: tests/golden/make_param_ab_golden.py)."""
    z = np.load(os.path.join(golden_dir, "param_ab_small.npz"))
    t = lambda n: torch.from_numpy(z[n])
    a, b = orc.param_ab_ref(t("beta"), t("k"), t("log_f"))
    assert a.shape == t("a").shape and b.shape == t("b").shape
    assert orc.rel_err(a, t("a")) < 1e-14 and orc.rel_err(b, t("b")) < 1e-14


def test_norm_gate_restatement_matches_the_reference_function(golden_dir):
    """``norm_gate_ref`` (forward and autograd gradients) against the reference's own ``normalize_torch`` called as the
    layer's epilogue calls it (tests/golden/make_norm_gate_golden.py; the reference computes in fp32)."""
    z = np.load(os.path.join(golden_dir, "norm_gate_small.npz"))
    leaves = [torch.from_numpy(z[n]).double().requires_grad_(True) for n in ("x", "gate", "weight")]
    o = orc.norm_gate_ref(*leaves, float(z["eps"]))
    grads = torch.autograd.grad((o * torch.from_numpy(z["d_o"]).double()).sum(), leaves)
    assert orc.rel_err(o, torch.from_numpy(z["o"])) < 1e-6
    for got, n in zip(grads, ("dx", "dgate", "dweight")):
        assert orc.rel_err(got, torch.from_numpy(z[n])) < 1e-5, n


def test_l2_norm_formula_matches_the_reference_function(golden_dir):
    """k / sqrt(sum_K k^2 + 1e-5) -- what HDLA_FLAG_NORM_K computes inside the operator and what the tests feed the
    oracle with -- against the reference's normalize_torch called as its l2_norm calls it."""
    z = np.load(os.path.join(golden_dir, "norm_gate_small.npz"))
    x = torch.from_numpy(z["x"]).double()
    assert orc.rel_err(x / torch.sqrt((x * x).sum(-1, keepdim=True) + 1e-5), torch.from_numpy(z["l2"])) < 1e-6


def test_oracle_score_matrices_match_the_reference_stage_test(golden_dir):
    """The four intra-chunk score matrices of the staged oracle against the torch reference block of the reference's own
    stage test, compute_A_ref_torch (test_fwd_A.py:10-62, called as at :203-214; tests/golden/make_stage_golden.py)."""
    z = np.load(os.path.join(golden_dir, "stage_A_small.npz"))
    t = lambda n: torch.from_numpy(z[n])
    B, T, H, K = t("q").shape
    C, R = int(z["chunk"]), 2
    st = orc.staged_forward(t("q"), t("k"), torch.zeros(B, T, H, 4, dtype=torch.float64), t("a"), t("b"), t("gk"), R, 1.0,
                            None, C)
    for n in ("Aqk", "Aqb", "Aak", "Aab"):
        mine = st[n].permute(0, 2, 3, 1, 4).reshape(t(n).shape)        # [B,H,NT,rows,cols] -> [B, NT*rows, H, cols]
        assert orc.rel_err(mine, t(n)) < 1e-12, n
    # the output stage: the reference's chunk_dplr_fwd_o_simple (test_fwd_o.py:9-94) on those score matrices
    st = orc.staged_forward(t("q"), t("k"), t("v"), t("a"), t("b"), t("gk"), R, 1.0, t("h0"), C)
    assert orc.rel_err(st["o_bthv"], t("o")) < 1e-12
