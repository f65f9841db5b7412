"""Seeded synthetic inputs with the value distributions of the benchmark configurations.

q, k ~ N(0,1), L2-normalised over K; v ~ N(0,1); for each rank component r:
a_r = -normalize(N(0,1)), b_r = normalize(N(0,1)) * sigmoid(N(0,1)) (one gate scalar per
(b,t,r,h)), interleaved time-major / rank-minor into ``[B, T*R, H, K]`` as the operator expects
(reference layout: HRDPLR/recurrent.py:66-67,96-97); gk = logsigmoid(N(0,1)) / gk_div per
``[B,T,H,K]`` (a log decay, <= 0); dO ~ N(0,1).  Everything is drawn in fp32 on the CPU from
one ``torch.Generator`` and then cast, so the same seed gives the same values on every device.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F


def make_inputs(B: int, T: int, H: int, K: int, V: int, R: int = 2, *, seed: int = 0,
                dtype: torch.dtype = torch.float32, device="cpu", gk_div: float = 16.0,
                h0_std: Optional[float] = None, with_dht: bool = False) -> Dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float32)
    q = F.normalize(rn(B, T, H, K), dim=-1)
    k = F.normalize(rn(B, T, H, K), dim=-1)
    v = rn(B, T, H, V)
    a = -F.normalize(rn(B, T, R, H, K), dim=-1)
    b = F.normalize(rn(B, T, R, H, K), dim=-1) * torch.sigmoid(rn(B, T, R, H, 1))
    a = a.reshape(B, T * R, H, K)
    b = b.reshape(B, T * R, H, K)
    gk = F.logsigmoid(rn(B, T, H, K)) / gk_div
    do = rn(B, T, H, V)
    out = dict(q=q, k=k, v=v, a=a, b=b, gk=gk, do=do)
    out = {n: x.to(dtype).to(device) for n, x in out.items()}
    if h0_std is not None:
        out["h0"] = (rn(B, H, K, V) * h0_std).to(device)
    if with_dht:
        out["dht"] = rn(B, H, K, V).to(device)
    return out
