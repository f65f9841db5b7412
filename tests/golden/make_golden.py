"""Generate the golden vectors in this folder from the reference's own ``HRDPLR/naive.py``.

Run once where the reference checkout is available::

    python tests/golden/make_golden.py /path/to/reference

``naive.py`` is loaded by file path (its package ``__init__`` pulls in optional dependencies),
run in fp64 on the CPU with ``scale=1.0`` (``naive.py`` never reads its ``scale`` argument), and
differentiated with ``torch.autograd.grad`` exactly as the reference's ``test_integrated.py:72-82``
does.  Two fixtures are written:

* ``naive_small.npz``  -- inputs and all outputs/gradients in full, B1 T64 H2 K32 V48, chunk 16
  and chunk 32 must agree, random initial state and dht, gk = logsigmoid(N(0,1)) (undivided).
* ``naive_cfg0.npz``   -- the CPU configuration B2 T256 H4 K=V=64 seed 0, zero initial state:
  a strided subsample (every 13th element) and the sum / abs-sum of every output and gradient,
  plus checksums of the seeded inputs so a test can tell a generator mismatch from a parity miss.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from hdla_impl_b200.synthetic import make_inputs  # noqa: E402


def load_naive(ref_root):
    spec = importlib.util.spec_from_file_location("ref_naive", os.path.join(ref_root, "HRDPLR", "naive.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def run_ref(m, x, R, chunk):
    names = ["q", "k", "v", "a", "b", "gk", "h0"]
    leaves = [x[n].double().clone().requires_grad_(True) for n in names]
    o, ht = m.hrdplr_naive(*leaves[:6], 1.0, leaves[6], True, R, False, chunk)
    loss = (o * x["do"].double()).sum() + (ht * x["dht"].double()).sum()
    grads = torch.autograd.grad(loss, leaves)
    out = {"o": o.detach(), "ht": ht.detach()}
    out.update({"d" + n: g for n, g in zip(names, grads)})
    return out


def main(ref_root):
    m = load_naive(ref_root)
    R = 2
    # ---- small, stored in full
    x = make_inputs(1, 64, 2, 32, 48, R, seed=7, gk_div=1.0, h0_std=1.0, with_dht=True)
    r16 = run_ref(m, x, R, 16)
    r32 = run_ref(m, x, R, 32)
    for n in r16:
        assert (r16[n] - r32[n]).abs().max() < 1e-10, n
    np.savez_compressed(os.path.join(HERE, "naive_small.npz"),
                        **{"in_" + n: t.numpy() for n, t in x.items()},
                        **{"out_" + n: t.numpy() for n, t in r16.items()})
    # ---- cfg0, subsampled
    x = make_inputs(2, 256, 4, 64, 64, R, seed=0, gk_div=16.0, h0_std=None, with_dht=True)
    x["h0"] = torch.zeros(2, 4, 64, 64)
    x["dht"] = torch.zeros(2, 4, 64, 64)
    r = run_ref(m, x, R, 64)
    r16 = run_ref(m, x, R, 16)
    for n in r:
        assert (r[n] - r16[n]).abs().max() < 1e-9, n
    rec = {}
    for n, t in x.items():
        rec["insum_" + n] = np.array([t.double().sum().item(), t.double().abs().sum().item()])
    for n, t in r.items():
        f = t.reshape(-1)
        rec["sub_" + n] = f[::13].numpy()
        rec["sum_" + n] = np.array([f.sum().item(), f.abs().sum().item(), f.abs().max().item()])
    np.savez_compressed(os.path.join(HERE, "naive_cfg0.npz"), **rec)
    print("written", os.listdir(HERE))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference-checkout")
    main(sys.argv[1])
