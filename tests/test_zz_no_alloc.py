"""GPU: hdla_chunk_fwd_noalloc -- the forward for callers that may not allocate device memory.

It runs the same kernels as hdla_chunk_fwd on a scratch array built into the library, so its
results must equal those of hdla_chunk_fwd with a torch-allocated workspace.  The file name makes
pytest collect it last: a run that stops at the first failure has then already run everything else.
Both calls go through the C ABI directly.  Two calls are made back to back on different inputs, so
a second call that wrongly depended on what the first left in the shared scratch would show.
"""
import ctypes as C

import pytest
import torch

from hdla_impl_b200.synthetic import make_inputs

pytestmark = pytest.mark.gpu
R = 2
NAMES = ("q", "k", "v", "a", "b", "gk")


def _dims(_lib, x, chunk):
    B, T, H, K = x["q"].shape
    return _lib.HdlaDims(B, T, H, K, x["v"].shape[-1], R, chunk, _lib.dtype_code(x["q"].dtype),
                         _lib.dtype_code(x["gk"].dtype), 0)


def _run_both(_lib, lib, x, chunk, dev):
    d = _dims(_lib, x, chunk)
    args = [x[n].to(dev).contiguous() for n in NAMES]
    h0 = x["h0"].to(dev).contiguous()
    B, T, H, K = x["q"].shape
    V = x["v"].shape[-1]
    scale = C.c_float(K ** -0.5)
    stream = _lib.stream_ptr(dev)
    outs = []
    for which in ("workspace", "noalloc"):
        o = torch.full_like(args[2], float("nan"))
        ht = torch.full((B, H, K, V), float("nan"), dtype=torch.float32, device=dev)
        if which == "workspace":
            n = lib.hdla_chunk_workspace_bytes(C.byref(d), 0)
            assert n > 0, _lib.last_error()
            ws = torch.empty(n, dtype=torch.uint8, device=dev)
            rc = lib.hdla_chunk_fwd(C.byref(d), *[_lib.ptr(t) for t in args], scale, _lib.ptr(h0), _lib.ptr(o),
                                    _lib.ptr(ht), _lib.ptr(ws), ws.numel(), stream)
        else:
            rc = lib.hdla_chunk_fwd_noalloc(C.byref(d), *[_lib.ptr(t) for t in args], scale, _lib.ptr(h0),
                                            _lib.ptr(o), _lib.ptr(ht), stream)
        assert rc == 0, f"{which}: {_lib.last_error()}"
        torch.cuda.synchronize(dev)
        outs.append((o.float().cpu(), ht.cpu()))
    return outs


@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 1e-4)])
def test_noalloc_forward_matches_workspace_forward_twice(dtype, tol):
    from hdla_impl_b200 import _lib
    from oracle import hdla_oracle as orc
    lib = _lib.load()
    dev = torch.device("cuda:0")
    with torch.cuda.device(dev):
        for call, (seed, T) in enumerate([(31, 256), (32, 192)]):       # two calls in a row, different inputs
            x = make_inputs(1, T, 2, 128, 128, R, seed=seed, dtype=dtype, h0_std=0.1)
            x["gk"] = x["gk"].float()
            (o_ws, ht_ws), (o_na, ht_na) = _run_both(_lib, lib, x, 64, dev)
            assert torch.isfinite(o_na).all() and torch.isfinite(ht_na).all()
            assert orc.rel_err(o_na, o_ws) < tol, f"call {call}: o"
            assert orc.rel_err(ht_na, ht_ws) < tol, f"call {call}: final state"


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    from hdla_impl_b200 import _lib
    lib = _lib.load()
    d = _lib.HdlaDims(8, 4096, 16, 128, 128, R, 64, 1, 0, 0)            # needs gigabytes of workspace
    rc = lib.hdla_chunk_fwd_noalloc(C.byref(d), None, None, None, None, None, None, C.c_float(1.0), None, None,
                                    None, None)
    assert rc == -3
    msg = _lib.last_error()
    assert "built-in scratch" in msg and "hdla_chunk_fwd" in msg
