"""``flash_qla.ops.gated_delta_rule.chunk`` (flash_qla/ops/gated_delta_rule/chunk/__init__.py:23-350): the
chunked prefill / training entry points, served by ``flashqla_b200.chunk``."""
from flashqla_b200.chunk import (ChunkGatedDeltaRuleFunction, chunk_gated_delta_rule, chunk_gated_delta_rule_bwd,
                                 chunk_gated_delta_rule_fwd)

__all__ = ["chunk_gated_delta_rule", "chunk_gated_delta_rule_fwd", "chunk_gated_delta_rule_bwd",
           "ChunkGatedDeltaRuleFunction"]
