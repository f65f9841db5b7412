"""Loader and timer for the reference's own ``hrdplr_naive`` (``HRDPLR/naive.py:76-263``) when
``oracle/install_ref.py`` has placed it under ``oracle/_ref/``.  TEST INFRASTRUCTURE ONLY: used by the
tests (to cross-check the restatement in ``hdla_oracle``) and by the benchmark's CPU-baseline legs,
never by the operator.
"""
from __future__ import annotations

import importlib.util
import os
import time
from typing import Optional

import torch

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "naive.py")
_mod = None


def available() -> bool:
    return os.path.isfile(_PATH)


def load():
    """The reference module, loaded by file path (its package ``__init__`` needs optional dependencies)."""
    global _mod
    if _mod is None:
        if not available():
            raise FileNotFoundError(f"{_PATH}: run oracle/install_ref.py with the reference checkout")
        spec = importlib.util.spec_from_file_location("hdla_ref_naive", _PATH)
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        _mod = m
    return _mod


def fwd_bwd(x: dict, R: int, chunk: int, dtype=torch.float32, h0: Optional[torch.Tensor] = None):
    """One forward + autograd backward of ``hrdplr_naive`` on the inputs ``x`` (q,k,v,a,b,gk,do), as the
    reference's own test does (``test_integrated.py:72-82``).  ``naive.py`` ignores ``scale`` and needs a tensor
    initial state and ``T % chunk == 0``.  Returns ``(o, final_state, grads)``."""
    m = load()
    names = ("q", "k", "v", "a", "b", "gk")
    lv = [x[n].to(dtype).clone().requires_grad_(True) for n in names]
    B, T, H, K = lv[0].shape
    V = lv[2].shape[-1]
    s0 = torch.zeros(B, H, K, V, dtype=dtype) if h0 is None else h0.to(dtype)
    o, ht = m.hrdplr_naive(*lv, 1.0, s0, True, R, False, chunk)
    grads = torch.autograd.grad((o * x["do"].to(dtype)).sum(), lv)
    return o.detach(), ht.detach(), grads


def time_fwd_bwd(x: dict, R: int, chunk: int, repeats: int = 3):
    """Best wall-clock seconds of ``repeats`` forward + backward passes in fp32 on all host threads."""
    torch.set_num_threads(os.cpu_count() or 1)
    best = None
    for _ in range(repeats):
        t0 = time.perf_counter()
        fwd_bwd(x, R, chunk)
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return best
