"""``flash_qla.ops`` (flash_qla/ops/__init__.py:4)."""
from .gated_delta_rule import chunk_gated_delta_rule

__all__ = ["chunk_gated_delta_rule"]
