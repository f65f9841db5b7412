"""hdla_impl_b200 -- the HDLA rank-2 DPLR delta-rule operator for NVIDIA B200 (sm_100a).

Drop-in for the operator entry points of the reference package (``HRDPLR/__init__.py:1-12``):
``chunk_hrdplr_delta_rule`` (chunked forward + backward, autograd) and
``fused_recurrent_dplr_delta_rule`` (fused recurrent forward).  PyTorch is only the host side:
every kernel is hand-written CUDA inside ``libhdla.so`` behind the C ABI of ``include/hdla.h``.
There is no CPU path and no fallback.
"""
from .hrdplr import ChunkDPLRDeltaRuleFunction, check_status, chunk_hrdplr_delta_rule, chunk_hrdplr_fwd
from .recurrent import (FusedRecurrentDPLRDeltaRuleFunction, fused_recurrent_dplr_delta_rule,
                        fused_recurrent_dplr_delta_rule_fwd)

__all__ = [
    "fused_recurrent_dplr_delta_rule",
    "chunk_hrdplr_delta_rule",
    "ChunkDPLRDeltaRuleFunction",
    "FusedRecurrentDPLRDeltaRuleFunction",
    "chunk_hrdplr_fwd",
    "check_status",
    "fused_recurrent_dplr_delta_rule_fwd",
]
