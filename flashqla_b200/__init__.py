"""flashqla_b200: B200 (sm_100a) gated-delta-rule kernels behind FlashQLA's Python API.

Public names follow the reference package (flash_qla/__init__.py:6-38).
"""
from .chunk import chunk_gated_delta_rule, chunk_gated_delta_rule_bwd, chunk_gated_delta_rule_fwd
from .graph import GraphedForward
from .handoff import prefill_into_state_pool
from .host_stream import chunk_gated_delta_rule_fwd_host
from .seq_parallel import chunk_gated_delta_rule_bwd_sp, chunk_gated_delta_rule_fwd_sp
from .recurrent import commit_verified_state, flashqla_recurrent_gdn_update, fused_sigmoid_gating_delta_rule_update
from .utils import check_device_status

__all__ = [
    "chunk_gated_delta_rule",
    "chunk_gated_delta_rule_fwd",
    "chunk_gated_delta_rule_bwd",
    "chunk_gated_delta_rule_fwd_host",
    "chunk_gated_delta_rule_fwd_sp",
    "chunk_gated_delta_rule_bwd_sp",
    "prefill_into_state_pool",
    "GraphedForward",
    "fused_sigmoid_gating_delta_rule_update",
    "flashqla_recurrent_gdn_update",
    "commit_verified_state",
    "check_device_status",
]
