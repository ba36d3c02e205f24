"""``flash_qla.ops.gated_delta_rule.recurrent_fused`` (recurrent_fused.py:6287-7537): decode / verify entry
points, served by ``flashqla_b200.recurrent``."""
from flashqla_b200.recurrent import flashqla_recurrent_gdn_update, fused_sigmoid_gating_delta_rule_update

__all__ = ["fused_sigmoid_gating_delta_rule_update", "flashqla_recurrent_gdn_update"]
