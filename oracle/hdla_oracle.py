"""CPU oracle for the HDLA rank-R DPLR delta-rule operator.  TEST INFRASTRUCTURE ONLY.

This module is the checker, never the product: only the tests, the smoke check and the
benchmark's CPU-baseline leg may import it.  The shipped operator never calls it and has no
CPU fallback.

It restates, in plain torch on the CPU (fp64 by default), the algorithm of the reference
project's operator path:

* ``recurrent_ref``  -- the per-token recurrence of ``HRDPLR/recurrent.py:75-115`` (one state
  ``S[K,V]`` per (sequence, head); both rank terms read ``S_{t-1}``; ``o_t = (scale*q_t)^T S_t``),
  including ``reverse`` and ``cu_seqlens``.
* ``chunked_ref``    -- the chunked formulation of ``HRDPLR/naive.py:76-263`` (chunk-local
  cumulative log-decays ``gi``/``ge``, the four intra-chunk matrices, the ``(I-Aab)^-1`` WY
  inverse, ``w``/``u``, the inter-chunk state loop), vectorised, differentiable by autograd.
  Unlike ``naive.py:83`` (which never reads ``scale``) it applies ``scale`` to ``q`` as the
  reference's kernels do (``HRDPLR/fwd_triton.py:222-245``).
* ``staged_forward`` / ``staged_backward`` -- every intermediate of the reference's stage
  sequence (``HRDPLR/hrdplr.py:25-99`` forward, ``:146-284`` backward; stage formulas as in
  ``HRDPLR/bwd_triton.py`` kernels dAu/dhu/dv/bwd_o/wy/intra/dgk) written as explicit tensor
  algebra.  These are the specification each CUDA stage is compared with.

Parity pin: ``tests/golden/`` holds outputs of the reference's own ``HRDPLR/naive.py``
(imported from the reference checkout, forward and autograd gradients) on seeded inputs;
``tests/test_oracle.py`` checks all three restatements against them.

Conventions: q,k,gk ``[B,T,H,K]``; v ``[B,T,H,V]``; a,b ``[B,T*R,H,K]`` with row ``t*R+r``;
state ``[B,H,K,V]``; ``gk`` is a log decay (<= 0).
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch


def _f(x: Optional[torch.Tensor], dtype) -> Optional[torch.Tensor]:
    return None if x is None else x.detach().to("cpu").to(dtype)


# --------------------------------------------------------------------------------------
# 1. per-token recurrence  (HRDPLR/recurrent.py:75-115)
# --------------------------------------------------------------------------------------
def recurrent_ref(q, k, v, a, b, gk, rank_ab: int, scale: Optional[float] = None,
                  initial_state=None, output_final_state: bool = True, reverse: bool = False,
                  cu_seqlens=None, dtype=torch.float64) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """S_t = diag(exp(g_t)) S_{t-1} + sum_r b_{t,r} (a_{t,r}^T S_{t-1}) + k_t v_t^T ; o_t = scale q_t^T S_t.

    Differentiable when the inputs require grad (no in-place writes on graph tensors).
    """
    B, T, H, K = q.shape
    V = v.shape[-1]
    R = rank_ab
    if scale is None:
        scale = K ** -0.5
    cast = (lambda x: x.to(dtype)) if q.requires_grad or v.requires_grad else (lambda x: _f(x, dtype))
    q, k, v, a, b, gk = map(cast, (q, k, v, a, b, gk))
    if cu_seqlens is None:
        bounds = [(n, 0, T) for n in range(B)]
    else:
        cs = [int(c) for c in cu_seqlens]
        assert B == 1
        bounds = [(0, cs[i], cs[i + 1]) for i in range(len(cs) - 1)]
    N = len(bounds)
    o_rows = [[None] * T for _ in range(B)]
    finals = []
    for n, (bi, bos, eos) in enumerate(bounds):
        if initial_state is not None:
            S = cast(initial_state)[n]
        else:
            S = torch.zeros(H, K, V, dtype=dtype)
        order = range(eos - 1, bos - 1, -1) if reverse else range(bos, eos)
        for t in order:
            contrib = 0
            for r in range(R):
                a_r = a[bi, t * R + r]                      # [H,K]
                b_r = b[bi, t * R + r]
                contrib = contrib + b_r[:, :, None] * torch.einsum("hk,hkv->hv", a_r, S)[:, None, :]
            S = torch.exp(gk[bi, t])[:, :, None] * S + contrib + k[bi, t][:, :, None] * v[bi, t][:, None, :]
            o_rows[bi][t] = torch.einsum("hk,hkv->hv", q[bi, t] * scale, S)
        finals.append(S)
    o = torch.stack([torch.stack([r if r is not None else torch.zeros(H, V, dtype=dtype) for r in rows])
                     for rows in o_rows])
    ht = torch.stack(finals) if output_final_state else None
    return o, ht


# --------------------------------------------------------------------------------------
# helpers for the chunked forms
# --------------------------------------------------------------------------------------
def _chunk_size(T: int, chunk_size: int) -> int:
    """BT = min(chunk_size, max(next_pow2(T), 16))   (HRDPLR/hrdplr.py:42)."""
    p2 = 1 << max(0, (T - 1).bit_length())
    return min(chunk_size, max(p2, 16))


def _pad_chunks(x: torch.Tensor, rows_per_tok: int, C: int) -> torch.Tensor:
    """[B, T*r, H, D] -> [B, H, NT, C*r, D], zero padded to a whole number of chunks."""
    B, TR, H, D = x.shape
    T = TR // rows_per_tok
    NT = (T + C - 1) // C
    pad = NT * C - T
    if pad:
        x = torch.cat([x, x.new_zeros(B, pad * rows_per_tok, H, D)], dim=1)
    return x.view(B, NT, C * rows_per_tok, H, D).permute(0, 3, 1, 2, 4)


def _unpad(x: torch.Tensor, rows_per_tok: int, T: int) -> torch.Tensor:
    """[B, H, NT, C*r, D] -> [B, T*r, H, D]."""
    B, H, NT, CR, D = x.shape
    return x.permute(0, 2, 3, 1, 4).reshape(B, NT * CR, H, D)[:, : T * rows_per_tok]


def _masks(C: int, R: int, device=None):
    i = torch.arange(C, device=device)
    ir = torch.arange(C * R, device=device) // R
    m_qk = (i[None, :] <= i[:, None])          # [C, C]      j <= i
    m_qb = (ir[None, :] <= i[:, None])         # [C, CR]
    m_ak = (i[None, :] < ir[:, None])          # [CR, C]     j <  i
    m_ab = (ir[None, :] < ir[:, None])         # [CR, CR]
    return m_qk, m_qb, m_ak, m_ab


def _gated_gram(x, gx, y, gy, mask):
    """A[i,j] = sum_k x[i,k] y[j,k] exp(gx[i,k]-gy[j,k]) on the mask, 0 elsewhere.

    The exponent is evaluated per (i,j,k) so it never overflows (it is <= 0 on the mask).
    x,gx: [...,m,K]; y,gy: [...,n,K]; mask [m,n].
    """
    d = gx[..., :, None, :] - gy[..., None, :, :]
    d = torch.where(mask[..., None], d, torch.zeros((), dtype=d.dtype))
    e = torch.exp(d) * mask[..., None].to(d.dtype)
    return torch.einsum("...ik,...jk,...ijk->...ij", x, y, e)


# --------------------------------------------------------------------------------------
# 2. staged forward: every intermediate of HRDPLR/hrdplr.py:25-99
# --------------------------------------------------------------------------------------
def staged_forward(q, k, v, a, b, gk, rank_ab: int, scale: float, initial_state=None,
                   chunk_size: int = 64, dtype=torch.float64, differentiable: bool = False
                   ) -> Dict[str, torch.Tensor]:
    """All stage intermediates, chunk-major ``[B,H,NT,rows,cols]`` (zero padded last chunk).

    keys: gi, ge, Aqk, Aqb, Aak, Aab, M, qg, kg, ag, bg, w, u, h (state entering each chunk,
    ``[B,H,NT,K,V]``), v2, o (chunk-major), o_bthv (``[B,T,H,V]``), ht, decay (exp(g_last)).
    """
    R = rank_ab
    B, T, H, K = q.shape
    V = v.shape[-1]
    C = _chunk_size(T, chunk_size)
    cast = (lambda x: x.to(dtype)) if differentiable else (lambda x: _f(x, dtype))
    q, k, v, a, b, gk = map(cast, (q, k, v, a, b, gk))
    qc, kc, vc, gc = (_pad_chunks(x, 1, C) for x in (q, k, v, gk))
    ac, bc = (_pad_chunks(x, R, C) for x in (a, b))
    NT = qc.shape[2]

    gi = gc.cumsum(-2)                                   # naive.py:107
    ge = gi - gc                                         # naive.py:108
    gi_ab = gi.repeat_interleave(R, dim=-2)
    ge_ab = ge.repeat_interleave(R, dim=-2)
    g_last = gi[..., -1:, :]                             # [B,H,NT,1,K]

    m_qk, m_qb, m_ak, m_ab = _masks(C, R)
    qs = qc * scale
    Aqk = torch.stack([_gated_gram(qs[:, :, n], gi[:, :, n], kc[:, :, n], gi[:, :, n], m_qk) for n in range(NT)], 2)
    Aqb = torch.stack([_gated_gram(qs[:, :, n], gi[:, :, n], bc[:, :, n], gi_ab[:, :, n], m_qb) for n in range(NT)], 2)
    Aak = torch.stack([_gated_gram(ac[:, :, n], ge_ab[:, :, n], kc[:, :, n], gi[:, :, n], m_ak) for n in range(NT)], 2)
    Aab = torch.stack([_gated_gram(ac[:, :, n], ge_ab[:, :, n], bc[:, :, n], gi_ab[:, :, n], m_ab) for n in range(NT)], 2)

    eye = torch.eye(C * R, dtype=dtype)
    # (I - Aab)^-1 : unit lower triangular (naive.py:189-192 does the same by row substitution)
    M = torch.linalg.solve_triangular(eye - Aab, eye.expand_as(Aab), upper=False)

    qg = qs * torch.exp(gi)
    kg = kc * torch.exp(g_last - gi)
    ag = ac * torch.exp(ge_ab)
    bg = bc * torch.exp(g_last - gi_ab)
    w = M @ ag                                           # naive.py:195
    u = M @ (Aak @ vc)                                   # naive.py:196
    decay = torch.exp(g_last.squeeze(-2))                # [B,H,NT,K]

    S = cast(initial_state) if initial_state is not None else torch.zeros(B, H, K, V, dtype=dtype)
    hs, v2s, os_ = [], [], []
    for n in range(NT):                                  # naive.py:232-255
        hs.append(S)
        v2 = w[:, :, n] @ S + u[:, :, n]
        os_.append(qg[:, :, n] @ S + Aqk[:, :, n] @ vc[:, :, n] + Aqb[:, :, n] @ v2)
        S = decay[:, :, n, :, None] * S + kg[:, :, n].transpose(-1, -2) @ vc[:, :, n] \
            + bg[:, :, n].transpose(-1, -2) @ v2
        v2s.append(v2)
    h = torch.stack(hs, 2)
    v2 = torch.stack(v2s, 2)
    o = torch.stack(os_, 2)
    return dict(gi=gi, ge=ge, Aqk=Aqk, Aqb=Aqb, Aak=Aak, Aab=Aab, M=M, qg=qg, kg=kg, ag=ag, bg=bg,
                w=w, u=u, h=h, v2=v2, o=o, o_bthv=_unpad(o, 1, T), ht=S, decay=decay,
                q=qc, k=kc, v=vc, a=ac, b=bc, g=gc, C=C, R=R, T=T, scale=scale)


def chunked_ref(q, k, v, a, b, gk, rank_ab: int, scale: Optional[float] = None, initial_state=None,
                output_final_state: bool = True, chunk_size: int = 64, dtype=torch.float64):
    """Chunked operator (HRDPLR/naive.py:76-263 with ``scale`` applied). Differentiable."""
    if scale is None:
        scale = q.shape[-1] ** -0.5
    st = staged_forward(q, k, v, a, b, gk, rank_ab, scale, initial_state, chunk_size, dtype,
                        differentiable=True)
    return st["o_bthv"], (st["ht"] if output_final_state else None)


# --------------------------------------------------------------------------------------
# 3. staged backward: explicit formulas of HRDPLR/hrdplr.py:146-284
# --------------------------------------------------------------------------------------
def staged_backward(st: Dict[str, torch.Tensor], do: torch.Tensor, dht: Optional[torch.Tensor] = None
                    ) -> Dict[str, torch.Tensor]:
    """Gradients and every backward intermediate from the forward intermediates ``st``.

    Stage names follow the reference's backward kernels (HRDPLR/bwd_triton.py):
    dAu (17-105), dhu (110-222), dv (227-290), bwd_o (295-487), wy (489-612), intra (614-883),
    dgk (885-947).  Returns dq,dk,dv,da,db,dgk in the public layouts, dh0, and chunk-major
    intermediates dAqk,dAqb,dAak,dAab,dv2,dh,dqg,dkg,dbg,dag,dw,dgk_last.
    """
    C, R, T, scale = st["C"], st["R"], st["T"], st["scale"]
    dtype = st["o"].dtype
    q, k, v, a, b = st["q"], st["k"], st["v"], st["a"], st["b"]
    gi, ge = st["gi"], st["ge"]
    B, H, NT = q.shape[:3]
    K, V = q.shape[-1], v.shape[-1]
    m_qk, m_qb, m_ak, m_ab = (m.to(dtype) for m in _masks(C, R))
    tr = lambda x: x.transpose(-1, -2)

    doc = _pad_chunks(_f(do, dtype), 1, C)                               # [B,H,NT,C,V]
    # --- dAu: gradients of the two output score matrices and the intra part of dv2
    dAqk = (doc @ tr(v)) * m_qk
    dAqb = (doc @ tr(st["v2"])) * m_qb
    dv2_intra = tr(st["Aqb"]) @ doc
    # --- dhu: reverse scan over chunks
    dS = _f(dht, dtype) if dht is not None else torch.zeros(B, H, K, V, dtype=dtype)
    dh = [None] * NT          # gradient of the state at the END of chunk n
    dv2 = [None] * NT
    for n in range(NT - 1, -1, -1):
        dh[n] = dS
        dv2[n] = dv2_intra[:, :, n] + st["bg"][:, :, n] @ dS
        dS = st["decay"][:, :, n, :, None] * dS + tr(st["qg"][:, :, n]) @ doc[:, :, n] \
            + tr(st["w"][:, :, n]) @ dv2[n]
    dh0 = dS
    dh = torch.stack(dh, 2)
    dv2 = torch.stack(dv2, 2)
    # --- dv (direct part)
    dv0 = st["kg"] @ dh + tr(st["Aqk"]) @ doc
    # --- bwd_o: gradients of the gated operands and of w
    h = st["h"]
    dqg = doc @ tr(h)
    dkg = v @ tr(dh)
    dbg = st["v2"] @ tr(dh)
    dw = dv2 @ tr(h)
    dgk_last = st["decay"] * (h * dh).sum(-1) + (st["kg"] * dkg).sum(-2) + (st["bg"] * dbg).sum(-2)
    # --- wy: through u = M (Aak v), w = M ag, M = (I - Aab)^-1
    M, Aak = st["M"], st["Aak"]
    P = Aak @ v
    dP = tr(M) @ dv2
    dAak = (dP @ tr(v)) * m_ak
    dv = dv0 + tr(Aak) @ dP
    dM = dv2 @ tr(P) + dw @ tr(st["ag"])
    dAab = (tr(M) @ dM @ tr(M)) * m_ab
    dag = tr(M) @ dw
    # --- intra: from score-matrix gradients to q,k,a,b (direct exponent differences)
    gi_ab = gi.repeat_interleave(R, dim=-2)
    ge_ab = ge.repeat_interleave(R, dim=-2)
    g_last = gi[..., -1:, :]

    def row_side(dA, gx, y, gy):      # dx[i,k] = sum_j dA[i,j] y[j,k] exp(gx[i,k]-gy[j,k])
        d = gx[..., :, None, :] - gy[..., None, :, :]
        e = torch.exp(torch.where(dA[..., None] != 0, d, torch.zeros((), dtype=dtype)))
        return torch.einsum("...ij,...jk,...ijk->...ik", dA, y, e)

    def col_side(dA, x, gx, gy):      # dy[j,k] = sum_i dA[i,j] x[i,k] exp(gx[i,k]-gy[j,k])
        d = gx[..., :, None, :] - gy[..., None, :, :]
        e = torch.exp(torch.where(dA[..., None] != 0, d, torch.zeros((), dtype=dtype)))
        return torch.einsum("...ij,...ik,...ijk->...jk", dA, x, e)

    qs = q * scale
    dqs = torch.zeros_like(q); dk = torch.zeros_like(k); da = torch.zeros_like(a); db = torch.zeros_like(b)
    for n in range(NT):
        s = (slice(None), slice(None), n)
        dqs[s] = row_side(dAqk[s], gi[s], k[s], gi[s]) + row_side(dAqb[s], gi[s], b[s], gi_ab[s])
        da[s] = row_side(dAak[s], ge_ab[s], k[s], gi[s]) + row_side(dAab[s], ge_ab[s], b[s], gi_ab[s])
        dk[s] = col_side(dAqk[s], qs[s], gi[s], gi[s]) + col_side(dAak[s], a[s], ge_ab[s], gi[s])
        db[s] = col_side(dAqb[s], qs[s], gi[s], gi_ab[s]) + col_side(dAab[s], a[s], ge_ab[s], gi_ab[s])
    dqs = dqs + dqg * torch.exp(gi)
    dk = dk + dkg * torch.exp(g_last - gi)
    da = da + dag * torch.exp(ge_ab)
    db = db + dbg * torch.exp(g_last - gi_ab)
    # --- dgk: d/d(log decay). row-side gates give +x*dx, column-side gates give -y*dy
    sum_r = lambda x: x.reshape(*x.shape[:-2], C, R, K).sum(-2)
    d_gi = qs * dqs - k * dk - sum_r(b * db)          # direct gradient w.r.t. inclusive cumsum
    d_ge = sum_r(a * da)                              # ... w.r.t. exclusive cumsum
    raw = d_gi + d_ge
    revcum = raw.flip(-2).cumsum(-2).flip(-2)
    dg = revcum - d_ge + dgk_last[..., None, :]
    dq = dqs * scale
    out = dict(dq=_unpad(dq, 1, T), dk=_unpad(dk, 1, T), dv=_unpad(dv, 1, T), da=_unpad(da, R, T),
               db=_unpad(db, R, T), dgk=_unpad(dg, 1, T), dh0=dh0,
               dAqk=dAqk, dAqb=dAqb, dAak=dAak, dAab=dAab, dv2=dv2, dv2_intra=dv2_intra, dh=dh, dqg=dqg,
               dkg=dkg, dbg=dbg, dag=dag, dw=dw, dgk_last=dgk_last, dv0=dv0)
    return out


def autograd_ref(fn, q, k, v, a, b, gk, h0, do, dht, dtype=torch.float64):
    """Run ``fn(q,k,v,a,b,gk,h0) -> (o, ht)`` in ``dtype`` on leaf copies and return
    (o, ht, dict of gradients) for loss = sum(o*do) + sum(ht*dht)."""
    leaves = [x.detach().to("cpu").to(dtype).requires_grad_(True) for x in (q, k, v, a, b, gk)]
    h0l = None if h0 is None else h0.detach().to("cpu").to(dtype).requires_grad_(True)
    o, ht = fn(*leaves, h0l)
    loss = (o * _f(do, dtype)).sum()
    if dht is not None and ht is not None:
        loss = loss + (ht * _f(dht, dtype)).sum()
    ins = leaves + ([h0l] if h0l is not None else [])
    grads = torch.autograd.grad(loss, ins)
    names = ["dq", "dk", "dv", "da", "db", "dgk"] + (["dh0"] if h0l is not None else [])
    return o.detach(), (None if ht is None else ht.detach()), dict(zip(names, grads))

# --------------------------------------------------------------------------------------
# 4. the layer's a/b parametrisation (HRDPLR/hdla_custom.py:19-43, which computes a and b and returns nothing)
# --------------------------------------------------------------------------------------
def param_ab_ref(beta: torch.Tensor, k: torch.Tensor, log_f: torch.Tensor):
    """``a, b`` of shape ``[B, 2T, H, K]`` (row ``2t + r``) as the reference's ``parameterize_a_b`` forms them:
    a1 = -beta k (:24), a2 = at2 + a1 sum_K(k at2) with at2 = -beta e^{log_f} k (:25-33), b1 = e^{log_f} k, b2 = k
    (:35-36), stacked rank-minor (:38-42).  Differentiable.  Pinned by tests/golden/param_ab_small.npz, whose a and b
    were read out of the reference function's own frame."""
    a_t1 = -beta * k
    a_t2 = -beta * torch.exp(log_f) * k
    a_2 = a_t2 + a_t1 * torch.sum(k * a_t2, dim=-1, keepdim=True)
    b_1 = torch.exp(log_f) * k
    B, T, H, K = k.shape
    a = torch.stack([a_t1, a_2], dim=2).reshape(B, 2 * T, H, K)
    b = torch.stack([b_1, k], dim=2).reshape(B, 2 * T, H, K)
    return a, b

def norm_gate_ref(x: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """The layer's output epilogue (HRDPLR/hdla_custom.py:341-345): ``normalize_torch``
    (HRDPLR/normalizations/normalize/normalize/normalize_torch.py:65-79) as ``RMSNormFusedGate`` calls it -- sigmoid
    gate applied before the norm (:65-68), no mean, one group, ``o = c y / sqrt(sum(y^2) + eps) * weight`` (:75-79) with
    ``c = sqrt(D)`` (HRDPLR/normalizations/utils.py, rmsnorm).  Differentiable.  Pinned by
    tests/golden/norm_gate_small.npz, which the reference function itself produced."""
    y = x * torch.sigmoid(gate)
    D = x.shape[-1]
    return (D ** 0.5) * y / torch.sqrt((y * y).sum(-1, keepdim=True) + eps) * weight


def rel_err(x: torch.Tensor, ref: torch.Tensor) -> float:
    """max|x-ref| / max|ref|  -- the parity metric used everywhere."""
    x = x.detach().to("cpu").to(torch.float64)
    ref = ref.detach().to("cpu").to(torch.float64)
    den = ref.abs().max().item()
    num = (x - ref).abs().max().item()
    if not math.isfinite(num):
        return float("inf")
    return num / den if den > 0 else num
