"""GPU: every intermediate of the tensor-core (bf16) forward pipeline against the fp64 oracle.

The bf16 pipeline works on operands scaled around half the chunk's total log decay
(Qh = scale q e^{gi-half}, Kh = k e^{half-gi}, Ah = a e^{ge-half}, Bh = b e^{half-gi}, E = e^{half});
the oracle's stage quantities are converted to that form here.  Tolerance 2e-2 of each tensor's max.
"""
import ctypes as C

import pytest
import torch

from oracle import hdla_oracle as orc
from hdla_impl_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu
R = 2


def _dump(ws, dims, name, shape, dev):
    from hdla_impl_b200 import _lib
    out = torch.empty(shape, dtype=torch.float32, device=dev)
    rc = _lib.load().hdla_debug_tc_buffer(C.byref(dims), _lib.ptr(ws), name.encode(), _lib.ptr(out),
                                          _lib.stream_ptr(dev))
    _lib.check(rc, "hdla_debug_tc_buffer")
    torch.cuda.synchronize()
    return out.cpu().double()


@pytest.mark.parametrize("fused", [False, True])          # four-kernel and one-kernel chunk preparation
@pytest.mark.parametrize("T,gk_div,h0_std", [(256, 16.0, None), (200, 2.0, 0.5), (320, 1.0, 0.5)])
def test_tc_forward_stages(T, gk_div, h0_std, fused, monkeypatch):
    from hdla_impl_b200 import _lib, hrdplr
    monkeypatch.setenv("HDLA_FUSED_PREP", "1" if fused else "0")
    dev = torch.device("cuda:0")
    B, H, K, V, Cc = 2, 2, 128, 128, 64
    x = make_inputs(B, T, H, K, V, R, seed=21, dtype=torch.bfloat16, gk_div=gk_div, h0_std=h0_std)
    x["gk"] = x["gk"].float()
    names = ("q", "k", "v", "a", "b", "gk")
    args = [x[n].to(dev) for n in names]
    scale = K ** -0.5
    h0 = None if h0_std is None else x["h0"].to(dev)
    o, ht, ws, _ = hrdplr._chunk_fwd(*args, scale, h0, True, R, False, Cc, _keep_ws=True)
    torch.cuda.synchronize()
    dims = hrdplr._dims(args[0], args[2], args[3], args[5], R, Cc)
    st = orc.staged_forward(*[x[n].double() for n in names], R, scale, None if h0_std is None else x["h0"], Cc)
    NT = st["gi"].shape[2]
    G = B * H * NT
    half = st["gi"][..., -1:, :] / 2
    rep = lambda t: t.repeat_interleave(R, dim=-2)
    E = torch.exp(half)
    want = {
        "Qh": (st["q"] * scale * torch.exp(st["gi"] - half), (64, 128)),
        "Kh": (st["k"] * torch.exp(half - st["gi"]), (64, 128)),
        "Ah": (st["a"] * torch.exp(rep(st["ge"]) - half), (128, 128)),
        "Bh": (st["b"] * torch.exp(half - rep(st["gi"])), (128, 128)),
        "Vc": (st["v"], (64, 128)),
        "Aqk": (st["Aqk"], (64, 64)), "Aqb": (st["Aqb"], (64, 128)), "Aak": (st["Aak"], (128, 64)),
        "M": (st["M"], (128, 128)),                      # Aab itself never leaves the SM: M = (I - Aab)^-1 covers it
        "P": (st["Aak"] @ st["v"], (128, 128)), "U": (st["u"], (128, 128)),
        "W": (st["w"] / E, (128, 128)),
        "Hs": (st["h"] * E.transpose(-1, -2), (128, 128)),
        "V2": (st["v2"], (128, 128)),
    }
    status = ws[:8].view(torch.int32).tolist()
    assert status == [0, 0], f"status words {status}"
    bad = []
    for n, (ref, shp) in want.items():
        got = _dump(ws, dims, n, (G,) + shp, dev).view(B, H, NT, *shp)
        e = orc.rel_err(got, ref)
        if not e < 2e-2:
            bad.append(f"{n}: {e:.3e}")
    e = orc.rel_err(o, st["o_bthv"])
    if not e < 2e-2:
        bad.append(f"o: {e:.3e}")
    e = orc.rel_err(ht, st["ht"])
    if not e < 2e-2:
        bad.append(f"ht: {e:.3e}")
    assert not bad, "; ".join(bad)


@pytest.mark.parametrize("fused", [False, True])
def test_tc_backward_stages(fused, monkeypatch):
    """Backward intermediates of the tensor-core pipeline (hat-operand form) against the oracle's stage formulas."""
    import hdla_impl_b200 as HD
    from hdla_impl_b200 import _lib, hrdplr
    monkeypatch.setenv("HDLA_FUSED_PREP", "1" if fused else "0")
    dev = torch.device("cuda:0")
    B, T, H, K, V, Cc = 1, 192, 2, 128, 128, 64
    x = make_inputs(B, T, H, K, V, R, seed=22, dtype=torch.bfloat16, gk_div=8.0, h0_std=0.3, with_dht=True)
    x["gk"] = x["gk"].float()
    names = ("q", "k", "v", "a", "b", "gk")
    args = [x[n].to(dev) for n in names]
    scale = K ** -0.5
    h0 = x["h0"].to(dev)
    o, ht, ws, _ = hrdplr._chunk_fwd(*args, scale, h0, True, R, False, Cc, _keep_ws=True)
    lib = _lib.load()
    dims = hrdplr._dims(args[0], args[2], args[3], args[5], R, Cc, _lib.FLAG_WS_HOLDS_FWD)
    do = x["do"].to(dev)
    dht = x["dht"].to(dev)
    outs = [torch.empty_like(t) for t in args]
    dh0 = torch.empty_like(h0)
    rc = lib.hdla_chunk_bwd(C.byref(dims), *[_lib.ptr(t) for t in args], C.c_float(scale), _lib.ptr(h0), _lib.ptr(do),
                            _lib.ptr(dht), *[_lib.ptr(t) for t in outs], _lib.ptr(dh0), _lib.ptr(ws), ws.numel(),
                            _lib.stream_ptr(dev))
    _lib.check(rc, "hdla_chunk_bwd")
    torch.cuda.synchronize()
    st = orc.staged_forward(*[x[n].double() for n in names], R, scale, x["h0"], Cc)
    g = orc.staged_backward(st, x["do"].double(), x["dht"])
    NT = st["gi"].shape[2]
    G = B * H * NT
    half = st["gi"][..., -1:, :] / 2
    E = torch.exp(half)                                   # [B,H,NT,1,K]
    Ecol = E.transpose(-1, -2)                            # scales state rows k
    want = {
        "dAqk": (g["dAqk"], (64, 64)), "dAqb": (g["dAqb"], (64, 128)),
        "DV2": (g["dv2"], (128, 128)),
        "DE": (g["dh"] * Ecol, (128, 128)),               # E (.) gradient of the state leaving the chunk
        "dW": (g["dw"] * E, (128, 128)),                  # gradient of Wh = w / E
        "dP": (st["M"].transpose(-1, -2) @ g["dv2"], (128, 128)),
        "dAak": (g["dAak"], (128, 64)), "dAab": (g["dAab"], (128, 128)),
    }
    bad = []
    for n, (ref, shp) in want.items():
        got = _dump(ws, dims, n, (G,) + shp, dev).view(B, H, NT, *shp)
        e = orc.rel_err(got, ref)
        if not e < 2e-2:
            bad.append(f"{n}: {e:.3e}")
    dgl = _dump(ws, dims, "dgl", (G, 128), dev).view(B, H, NT, 128)
    e = orc.rel_err(dgl, g["dgk_last"])
    if not e < 2e-2:
        bad.append(f"dgl: {e:.3e}")
    for t, n in zip(outs + [dh0], ["dq", "dk", "dv", "da", "db", "dgk", "dh0"]):
        e = orc.rel_err(t, g[n])
        if not e < 2e-2:
            bad.append(f"{n}: {e:.3e}")
    assert not bad, "; ".join(bad)
