"""``flash_qla.utils`` names used by the reference's callers (flash_qla/utils/__init__.py:4-19), served by
``flashqla_b200.utils``."""
from flashqla_b200.utils import (fill_last_chunk_of_g, l2norm, pack, pad_and_reshape, prepare_chunk_indices,
                                 prepare_chunk_offsets, profile, unpack)

__all__ = ["profile", "pad_and_reshape", "pack", "unpack", "fill_last_chunk_of_g", "l2norm",
           "prepare_chunk_indices", "prepare_chunk_offsets"]
