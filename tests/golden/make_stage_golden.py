"""Generate ``stage_A_small.npz`` from the torch reference blocks of the reference's own stage tests:
``compute_A_ref_torch`` (test_fwd_A.py:10-62), called with the arguments that test uses for the four intra-chunk
score matrices (test_fwd_A.py:203-214), and ``chunk_dplr_fwd_o_simple`` (test_fwd_o.py:9-94), the output stage, fed
with those score matrices and with the gated queries, checkpoints and v2 of the staged oracle on the same inputs.

Run once where the reference checkout is available::

    python tests/golden/make_stage_golden.py /path/to/reference

The test file imports the Triton kernels at module level and cannot be imported without a GPU; the function's own
source text is taken out of the file (``ast``) and run as it stands, in fp64 on the CPU, on seeded inputs with the
chunk-local cumulative sums formed the way the test forms them (test_fwd_A.py:105-114).
"""
import ast
import os
import sys

import numpy as np
import torch
import triton

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import hdla_oracle as orc  # noqa: E402


def load_fn(path, name, ns):
    tree = ast.parse(open(path).read(), filename=path)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == name)
    exec(compile(ast.Module(body=[fn], type_ignores=[]), path, "exec"), ns)
    return ns[name]


def main():
    ref_root = sys.argv[1]
    compute_A = load_fn(os.path.join(ref_root, "test_fwd_A.py"), "compute_A_ref_torch", {"torch": torch})
    g = torch.Generator().manual_seed(21)
    B, T, H, K, BT, R = 1, 32, 2, 8, 16, 2
    rn = lambda *s: torch.randn(*s, generator=g, dtype=torch.float64)
    q, k, a, b = rn(B, T, H, K), rn(B, T, H, K), rn(B, T * R, H, K), rn(B, T * R, H, K)
    gk = torch.log(torch.sigmoid(rn(B, T, H, K)))
    gi = torch.zeros_like(gk)
    for i_t in range(T // BT):
        gi[:, i_t * BT:(i_t + 1) * BT] = torch.cumsum(gk[:, i_t * BT:(i_t + 1) * BT], dim=1)
    ge = gi - gk
    gi_ab = torch.repeat_interleave(gi, repeats=R, dim=1)
    ge_ab = torch.repeat_interleave(ge, repeats=R, dim=1)
    Aqk = compute_A(operand_a_in=q, operand_b_in=k, g_in=gi, gi_in=gi, rank_a=1, rank_b=1, BT=BT, USE_A=False)
    Aqb = compute_A(operand_a_in=q, operand_b_in=b, g_in=gi, gi_in=gi, rank_a=1, rank_b=R, BT=BT, USE_A=False)
    Aak = compute_A(operand_a_in=a, operand_b_in=k, g_in=ge_ab, gi_in=gi_ab, rank_a=R, rank_b=1, BT=BT, USE_A=True)
    Aab = compute_A(operand_a_in=a, operand_b_in=b, g_in=ge_ab, gi_in=gi_ab, rank_a=R, rank_b=R, BT=BT, USE_A=True)
    # output stage: o = qg h + tril(Aqk) v + mask(Aqb) v2 per chunk
    out_stage = load_fn(os.path.join(ref_root, "test_fwd_o.py"), "chunk_dplr_fwd_o_simple",
                        {"torch": torch, "triton": triton})
    V = 12
    v, h0 = rn(B, T, H, V), 0.3 * rn(B, H, K, V)
    st = orc.staged_forward(q, k, v, a, b, gk, R, 1.0, h0, BT)
    flat = lambda t: t.permute(0, 2, 3, 1, 4).reshape(B, -1, H, t.shape[-1])     # chunk-major -> [B, rows, H, D]
    o = out_stage(flat(st["qg"]), v, flat(st["v2"]), Aqk, Aqb, st["h"].permute(0, 2, 1, 3, 4).contiguous(), BT, R)
    np.savez_compressed(os.path.join(HERE, "stage_A_small.npz"), q=q.numpy(), k=k.numpy(), a=a.numpy(), b=b.numpy(),
                        gk=gk.numpy(), chunk=np.int64(BT), Aqk=Aqk.numpy(), Aqb=Aqb.numpy(), Aak=Aak.numpy(),
                        Aab=Aab.numpy(), v=v.numpy(), h0=h0.numpy(), o=o.numpy())
    print({n: tuple(t.shape) for n, t in dict(Aqk=Aqk, Aqb=Aqb, Aak=Aak, Aab=Aab).items()})


if __name__ == "__main__":
    main()
