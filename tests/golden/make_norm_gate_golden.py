"""Generate ``norm_gate_small.npz`` from the reference's own ``normalize_torch``
(HRDPLR/normalizations/normalize/normalize/normalize_torch.py:9-109), called the way the layer's output epilogue
calls it: ``RMSNormFusedGate`` (HRDPLR/normalizations/rms_norm.py:48-91) -> ``NormOp("rmsnorm")``
(HRDPLR/normalizations/utils.py: ``c = dim ** 0.5``, no mean, one group) with a sigmoid gate applied before the norm.

Run once where the reference checkout is available::

    python tests/golden/make_norm_gate_golden.py /path/to/reference

The module imports ``xopes.ops.act.act_torch`` (third-party package ``xopes``, not pinned by the reference, not
installed here); ``act_torch(x, "sigmoid")`` is the only use on this path and is stood in for by ``torch.sigmoid``.
Everything else executed is the reference function's own source text, taken out of the file with ``ast`` and run on
fp32 inputs (the function computes in fp32: ``x = x.float()``).  Outputs: o and, by autograd on the
reference function, the gradients of x, gate and weight for a fixed dO; and ``l2``, the same function as the layer's
``l2_norm`` calls it.
"""
import ast
import os
import sys
from typing import Optional, Tuple

import numpy as np
import torch
from einops import rearrange

HERE = os.path.dirname(os.path.abspath(__file__))


def load_normalize_torch(ref_root):
    path = os.path.join(ref_root, "HRDPLR", "normalizations", "normalize", "normalize", "normalize_torch.py")
    tree = ast.parse(open(path).read(), filename=path)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "normalize_torch")

    def act_torch(x, act):
        assert act == "sigmoid", act
        return torch.sigmoid(x)

    ns = {"torch": torch, "rearrange": rearrange, "Optional": Optional, "Tuple": Tuple, "act_torch": act_torch}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), path, "exec"), ns)
    return ns["normalize_torch"]


def main():
    fn = load_normalize_torch(sys.argv[1])
    g = torch.Generator().manual_seed(12)
    rows, D, eps = 7, 64, 1e-5
    x = torch.randn(rows, D, generator=g).requires_grad_(True)
    gate = torch.randn(rows, D, generator=g).requires_grad_(True)
    w = (1 + 0.1 * torch.randn(D, generator=g)).requires_grad_(True)
    do = torch.randn(rows, D, generator=g)
    o = fn(x, weight=w, gate=gate, gate_act="sigmoid", gate_pos="pre", c=D ** 0.5, eps=eps, use_mean=False,
           num_groups=1)
    dx, dg, dw = torch.autograd.grad((o * do).sum(), [x, gate, w])
    # the layer's l2_norm of k (HRDPLR/normalizations/l2_norm.py:4-14): the same function with c = 1, eps = 1e-5, no
    # weight, no gate
    l2 = fn(x.detach(), weight=None, bias=None, residual=None, c=1, eps=1e-5, use_mean=False, num_groups=1)
    np.savez_compressed(os.path.join(HERE, "norm_gate_small.npz"), x=x.detach().numpy(), gate=gate.detach().numpy(),
                        weight=w.detach().numpy(), d_o=do.numpy(), eps=np.float64(eps), o=o.detach().numpy(),
                        dx=dx.numpy(), dgate=dg.numpy(), dweight=dw.numpy(), l2=l2.numpy())
    print("o", tuple(o.shape), float(o.detach().abs().max()))


if __name__ == "__main__":
    main()
