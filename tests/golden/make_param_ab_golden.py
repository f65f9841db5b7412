"""Generate ``param_ab_small.npz`` from the reference's own ``parameterize_a_b`` (HRDPLR/hdla_custom.py:19-43).

Run once where the reference checkout is available::

    python tests/golden/make_param_ab_golden.py /path/to/reference

The layer module cannot be imported (its package pulls in dependencies that are not installed), and the function
computes ``a`` and ``b`` but has no return statement.  So the function's own source text is taken out of the file
(``ast``), compiled as it stands without its ``torch.compile`` decorator, run in fp64 on the CPU, and its local
variables ``a`` and ``b`` are read from its frame when it returns (``sys.setprofile``): the values stored are
computed by the reference's lines, not by a restatement.
"""
import ast
import os
import sys

import numpy as np
import torch
from einops import rearrange

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_locals(ref_root, beta, k, log_f):
    path = os.path.join(ref_root, "HRDPLR", "hdla_custom.py")
    tree = ast.parse(open(path).read(), filename=path)
    fn = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "parameterize_a_b")
    fn.decorator_list = []
    ns = {"torch": torch, "rearrange": rearrange}
    exec(compile(ast.Module(body=[fn], type_ignores=[]), path, "exec"), ns)
    grabbed = {}

    def prof(frame, event, arg):
        if event == "return" and frame.f_code.co_name == "parameterize_a_b":
            grabbed.update({n: frame.f_locals[n] for n in ("a", "b")})

    sys.setprofile(prof)
    try:
        ns["parameterize_a_b"](beta, k, log_f)
    finally:
        sys.setprofile(None)
    return grabbed["a"], grabbed["b"]


def main():
    ref_root = sys.argv[1]
    g = torch.Generator().manual_seed(11)
    B, T, H, K = 2, 5, 3, 16
    k = torch.nn.functional.normalize(torch.randn(B, T, H, K, generator=g, dtype=torch.float64), dim=-1)
    beta = 2 * torch.sigmoid(torch.randn(B, T, H, 1, generator=g, dtype=torch.float64))
    log_f = torch.nn.functional.logsigmoid(torch.randn(B, T, H, K, generator=g, dtype=torch.float64))
    a, b = reference_locals(ref_root, beta, k, log_f)
    np.savez_compressed(os.path.join(HERE, "param_ab_small.npz"), beta=beta.numpy(), k=k.numpy(), log_f=log_f.numpy(),
                        a=a.numpy(), b=b.numpy())
    print("a", tuple(a.shape), "b", tuple(b.shape))


if __name__ == "__main__":
    main()
