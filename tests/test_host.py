"""CPU: the C-ABI library loads and exports every declared symbol; host-side validation."""
import ctypes as C
import os
import re

import pytest
import torch

from hdla_impl_b200 import _lib
from hdla_impl_b200.synthetic import make_inputs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    hdr = open(os.path.join(ROOT, "include", "hdla.h")).read()
    declared = set()
    for name in ("hdla.h", "hdla_debug.h"):            # the operator's C ABI and the instrumentation / test hooks
        found = set(re.findall(r"HDLA_API[^;(]*?\b(hdla_\w+)\s*\(", open(os.path.join(ROOT, "include", name)).read()))
        assert found, f"no declarations found in include/{name}"
        declared |= found
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in hdla.h but not exported"
    assert set(_lib.EXPORTS) == declared
    assert lib.hdla_version() == int(re.search(r"#define HDLA_VERSION (\d+)", hdr).group(1))


def test_workspace_query_and_error_text():
    lib = _lib.load()
    d = _lib.HdlaDims(2, 256, 4, 64, 64, 2, 64, 0, 0, 0)
    fwd = lib.hdla_chunk_workspace_bytes(C.byref(d), 0)
    both = lib.hdla_chunk_workspace_bytes(C.byref(d), 1)
    assert 0 < fwd < both
    d = _lib.HdlaDims(2, 256, 4, 64, 64, 2, 48, 0, 0, 0)
    assert lib.hdla_chunk_workspace_bytes(C.byref(d), 0) == 0
    assert "power of two" in _lib.last_error()
    d = _lib.HdlaDims(2, 0, 4, 64, 64, 2, 64, 0, 0, 0)
    assert lib.hdla_chunk_workspace_bytes(C.byref(d), 0) == 0
    assert "non-positive" in _lib.last_error()


def test_null_pointers_are_rejected_without_touching_a_gpu():
    lib = _lib.load()
    d = _lib.HdlaDims(1, 16, 1, 16, 16, 2, 16, 0, 0, 0)
    rc = lib.hdla_chunk_fwd(C.byref(d), None, None, None, None, None, None, 1.0, None, None, None, None, 0, None)
    assert rc == -1 and "null" in _lib.last_error()
    rc = lib.hdla_recurrent_fwd(C.byref(d), None, None, None, None, None, None, 1.0, None, None, None, None, 0, 0, None)
    assert rc == -1


def test_no_cpu_fallback():
    import hdla_impl_b200 as H
    x = make_inputs(1, 16, 1, 16, 16, 2, seed=0)
    args = [x[n] for n in ("q", "k", "v", "a", "b", "gk")]
    with pytest.raises(RuntimeError, match="CUDA"):
        H.chunk_hrdplr_delta_rule(*args, 2)
    with pytest.raises(RuntimeError, match="CUDA"):
        H.fused_recurrent_dplr_delta_rule(*args, 2)


def test_recurrent_argument_validation():
    import hdla_impl_b200 as H
    x = make_inputs(2, 8, 1, 16, 16, 2, seed=0)
    args = [x[n] for n in ("q", "k", "v", "a", "b", "gk")]
    with pytest.raises(ValueError, match="batch size"):
        H.fused_recurrent_dplr_delta_rule(*args, 2, cu_seqlens=torch.tensor([0, 8]))
    with pytest.raises(AssertionError):
        H.fused_recurrent_dplr_delta_rule(*args, 3)
    with pytest.raises(ValueError, match="4 dimensions"):
        H.fused_recurrent_dplr_delta_rule(args[0], args[1], args[2], args[3][0], args[4], args[5], 2)


def test_dtype_codes():
    assert _lib.dtype_code(torch.float32) == 0 and _lib.dtype_code(torch.bfloat16) == 1
    with pytest.raises(TypeError):
        _lib.dtype_code(torch.float16)


def test_numa_binding_is_best_effort_and_restores_affinity():
    import os
    from hdla_impl_b200.host import _parse_cpulist, numa_local_to
    assert _parse_cpulist("0-3,8,10-11\n") == {0, 1, 2, 3, 8, 10, 11}
    assert _parse_cpulist("") == set()
    before = os.sched_getaffinity(0)
    with numa_local_to("cuda:0") as nb:         # no GPU here: nothing to bind to, nothing changes
        inside = os.sched_getaffinity(0)
        assert nb.node is None or inside <= before
    assert os.sched_getaffinity(0) == before


def test_packed_batch_dims_are_validated_on_the_host():
    """cu_seqlens travels in HdlaDims as a HOST array: the workspace query sizes the plan from it and rejects
    offsets that do not rise from 0 to T, B != 1, and problems outside the tensor-core pipeline."""
    lib = _lib.load()
    d = _lib.HdlaDims(1, 598, 2, 128, 128, 2, 64, 1, 0, 0).with_seqlens([0, 200, 264, 597, 598])
    packed = lib.hdla_chunk_workspace_bytes(C.byref(d), 1)
    assert packed > 0, _lib.last_error()
    # 4 + 1 + 6 + 1 = 12 chunks against 10 for one sequence of 598 tokens: the packed plan is larger
    plain = lib.hdla_chunk_workspace_bytes(C.byref(_lib.HdlaDims(1, 598, 2, 128, 128, 2, 64, 1, 0, 0)), 1)
    assert packed > plain
    d = _lib.HdlaDims(1, 598, 2, 128, 128, 2, 64, 1, 0, 0).with_seqlens([0, 300, 200, 598])
    assert lib.hdla_chunk_workspace_bytes(C.byref(d), 1) == 0 and "decrease" in _lib.last_error()
    d = _lib.HdlaDims(1, 598, 2, 128, 128, 2, 64, 1, 0, 0).with_seqlens([0, 300, 500])
    assert lib.hdla_chunk_workspace_bytes(C.byref(d), 1) == 0 and "end at T" in _lib.last_error()
    d = _lib.HdlaDims(2, 598, 2, 128, 128, 2, 64, 1, 0, 0).with_seqlens([0, 598])
    assert lib.hdla_chunk_workspace_bytes(C.byref(d), 1) == 0 and "B == 1" in _lib.last_error()
    d = _lib.HdlaDims(1, 598, 2, 128, 128, 2, 64, 0, 0, 0).with_seqlens([0, 598])          # fp32: no packed path
    assert lib.hdla_chunk_workspace_bytes(C.byref(d), 1) == 0 and "tensor-core" in _lib.last_error()


def test_tensor_core_pipeline_selection():
    """bf16, rank 2, chunk 64 and head dims that are multiples of 8 up to 128 run on the tcgen05 pipeline."""
    lib = _lib.load()
    uses = lambda *a: lib.hdla_chunk_uses_tensor_cores(C.byref(_lib.HdlaDims(*a)))
    assert uses(2, 256, 2, 128, 128, 2, 64, 1, 0, 0) == 1
    assert uses(2, 256, 2, 64, 64, 2, 64, 1, 0, 0) == 1
    assert uses(2, 256, 2, 96, 48, 2, 64, 1, 1, 0) == 1
    assert uses(2, 256, 2, 100, 64, 2, 64, 1, 0, 0) == 0          # not a multiple of 8
    assert uses(2, 256, 2, 256, 128, 2, 64, 1, 0, 0) == 0         # beyond 128
    assert uses(2, 256, 2, 128, 128, 2, 16, 1, 0, 0) == 0         # chunk 16: fp32 pipeline
    assert uses(2, 256, 2, 128, 128, 2, 64, 0, 0, 0) == 0         # fp32 inputs
    assert uses(2, 256, 2, 128, 128, 2, 64, 1, 0, _lib.FLAG_FORCE_SIMT) == 0
    assert uses(2, 256, 2, 64, 64, 2, 64, 1, 0, _lib.PHASE_PRE) == 0      # phased calls need the full 128 x 128


def test_in_operator_parametrisation_flag_is_sized_and_gated_on_the_host():
    """HDLA_FLAG_PARAM_AB: the backward workspace grows by the two gradient tensors [B, 2T, H, K] bf16 that stay inside
    the library, the forward workspace does not change, and problems outside the tensor-core pipeline are refused."""
    lib = _lib.load()
    B, T, H, K = 2, 256, 2, 128
    plain = _lib.HdlaDims(B, T, H, K, 128, 2, 64, 1, 0, 0)
    fused = _lib.HdlaDims(B, T, H, K, 128, 2, 64, 1, 0, _lib.FLAG_PARAM_AB)
    assert lib.hdla_chunk_workspace_bytes(C.byref(fused), 0) == lib.hdla_chunk_workspace_bytes(C.byref(plain), 0)
    grow = lib.hdla_chunk_workspace_bytes(C.byref(fused), 1) - lib.hdla_chunk_workspace_bytes(C.byref(plain), 1)
    assert grow == 2 * B * 2 * T * H * K * 2
    fp32 = _lib.HdlaDims(B, T, H, K, 128, 2, 64, 0, 0, _lib.FLAG_PARAM_AB)
    assert lib.hdla_chunk_workspace_bytes(C.byref(fp32), 1) == 0 and "HDLA_FLAG_PARAM_AB" in _lib.last_error()
    # with the one-kernel preparation requested as well, the four-kernel layout is planned (that kernel reads a and b)
    both = _lib.HdlaDims(B, T, H, K, 128, 2, 64, 1, 0, _lib.FLAG_PARAM_AB | _lib.FLAG_FUSED_PREP)
    assert lib.hdla_chunk_workspace_bytes(C.byref(both), 1) == lib.hdla_chunk_workspace_bytes(C.byref(fused), 1)
    # normalising k inside the operator is part of the in-operator parametrisation
    alone = _lib.HdlaDims(B, T, H, K, 128, 2, 64, 1, 0, _lib.FLAG_NORM_K)
    assert lib.hdla_chunk_workspace_bytes(C.byref(alone), 1) == 0 and "HDLA_FLAG_PARAM_AB" in _lib.last_error()
    with_norm = _lib.HdlaDims(B, T, H, K, 128, 2, 64, 1, 0, _lib.FLAG_PARAM_AB | _lib.FLAG_NORM_K)
    assert lib.hdla_chunk_workspace_bytes(C.byref(with_norm), 1) == lib.hdla_chunk_workspace_bytes(C.byref(fused), 1)
