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


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_noalloc_forward_matches_workspace_forward_twice(dtype):
    """Same kernels, same inputs, only the scratch differs: the results must be equal bit for bit (the tolerance
    of this comparison is zero).  The second call is smaller and ends in a ragged chunk (200 = 3 * 64 + 8), so
    the zero padding of its last chunk is written over what the first, larger call left in the shared array."""
    from hdla_impl_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    with torch.cuda.device(dev):
        for call, (seed, T) in enumerate([(31, 256), (32, 200)]):       # two calls in a row, different inputs
            x = make_inputs(1, T, 2, 128, 128, R, seed=seed, dtype=dtype, h0_std=0.1)
            x["gk"] = x["gk"].float()
            (o_ws, ht_ws), (o_na, ht_na) = _run_both(_lib, lib, x, 64, dev)
            assert torch.isfinite(o_na).all() and torch.isfinite(ht_na).all()
            assert torch.equal(o_na, o_ws), f"call {call}: o"
            assert torch.equal(ht_na, ht_ws), f"call {call}: final state"


def test_noalloc_status_words_can_be_read_back():
    """Callers of the no-allocation entry point have no workspace pointer to read the kernels' status words
    from; hdla_noalloc_read_status copies them out of the built-in array.  A chunk decay beyond the bf16
    pipeline's range (64 tokens x 3 = 192 > 150) must show in word 1, a mild one must not."""
    from hdla_impl_b200 import _lib
    lib = _lib.load()
    dev = torch.device("cuda:0")
    with torch.cuda.device(dev):
        words = torch.zeros(3, dtype=torch.int32, device=dev)
        for gk_value, want in ((-3.0, 1), (-0.05, 0)):
            x = make_inputs(1, 128, 1, 128, 128, R, seed=33, dtype=torch.bfloat16)
            x["gk"] = torch.full_like(x["gk"].float(), gk_value)
            d = _dims(_lib, x, 64)
            args = [x[n].to(dev).contiguous() for n in NAMES]
            o = torch.empty_like(args[2])
            rc = lib.hdla_chunk_fwd_noalloc(C.byref(d), *[_lib.ptr(t) for t in args], C.c_float(128 ** -0.5), None,
                                            _lib.ptr(o), None, _lib.stream_ptr(dev))
            assert rc == 0, _lib.last_error()
            rc = lib.hdla_noalloc_read_status(_lib.ptr(words), _lib.stream_ptr(dev))
            assert rc == 0, _lib.last_error()
            torch.cuda.synchronize(dev)
            w = words.tolist()
            assert w[0] == 0 and w[1] == want, w
            seen = words[2:3].view(torch.float32).item()
            assert abs(seen - 64 * abs(gk_value)) < 1e-2 * 64 * abs(gk_value), seen


def test_noalloc_rejects_null_dims_as_invalid():
    from hdla_impl_b200 import _lib
    lib = _lib.load()
    rc = lib.hdla_chunk_fwd_noalloc(None, None, None, None, None, None, None, C.c_float(1.0), None, None, None, None)
    assert rc == -1 and "dims is null" in _lib.last_error()


def test_noalloc_rejects_problems_beyond_the_builtin_scratch():
    from hdla_impl_b200 import _lib
    lib = _lib.load()
    d = _lib.HdlaDims(8, 4096, 16, 128, 128, R, 64, 1, 0, 0)            # needs gigabytes of workspace
    rc = lib.hdla_chunk_fwd_noalloc(C.byref(d), None, None, None, None, None, None, C.c_float(1.0), None, None,
                                    None, None)
    assert rc == -3
    msg = _lib.last_error()
    assert "built-in scratch" in msg and "hdla_chunk_fwd" in msg
