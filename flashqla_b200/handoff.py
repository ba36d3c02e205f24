"""Prefill -> decode hand-off through the recurrent op's state pool.

The chunked forward keeps a sequence's state as ``[N, Hv, K, V]`` (``[N, Hv, V, K]`` with
``transpose_state_layout``, flash_qla/ops/gated_delta_rule/chunk/__init__.py:23-86); the recurrent op owns a
slot-indexed pool ``[slots, Hv, V, K]`` fp32 that it updates in place
(``fused_sigmoid_gating_delta_rule_update``, recurrent_fused.py:6287-6311).  A serving loop prefills a batch of
(new or continued) requests and then decodes them token by token from that pool; the reference leaves the
gather of the slots before the prefill and the scatter behind it to its caller.  Here the forward kernels take
the slot indices themselves (``initial_state_indices`` / ``final_state_indices`` of
``chunk_gated_delta_rule_fwd``), with the pool's layout and slot conventions: ``-1`` = no slot (zero state in,
nothing written back).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .chunk import chunk_gated_delta_rule_fwd


def prefill_into_state_pool(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    state_pool: torch.Tensor,
    state_indices: torch.Tensor,
    scale: Optional[float] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    continue_from_pool: bool = False,
    **forward_kwargs,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunked forward of ``N`` sequences whose final states land in ``state_pool[state_indices[n]]``
    (``[slots, Hv, V, K]`` fp32, contiguous, updated in place).  With ``continue_from_pool`` the sequences
    start from the states already in their slots (chunked prefill of a long prompt, prefix reuse), else from
    zero.  A slot index of ``-1`` starts from zero and writes nothing.  The pool may be fp32 or bf16.  Returns
    ``(o, state_pool)``.  ``forward_kwargs`` go to ``chunk_gated_delta_rule_fwd``
    (``use_qk_l2norm_in_kernel``, ``A_log`` ...)."""
    if state_pool.dim() != 4 or state_pool.dtype not in (torch.float32, torch.bfloat16) or not state_pool.is_contiguous():
        raise ValueError("state_pool must be a contiguous float32 or bfloat16 tensor [slots, Hv, V, K]")
    Hv = v.shape[2]
    if state_pool.shape[1] != Hv or tuple(state_pool.shape[2:]) != (128, 128):
        raise ValueError(f"state_pool must be [slots, {Hv}, 128, 128], got {tuple(state_pool.shape)}")
    N = q.shape[0] if cu_seqlens is None else cu_seqlens.numel() - 1
    if state_indices.numel() != N:
        raise ValueError(f"state_indices must have one entry per sequence ({N}), got {state_indices.numel()}")
    # The kernels index the pool themselves: a sequence reads its slot when it starts and writes it when it ends
    # (slots of different sequences must differ), so nothing is gathered or scattered around the call.
    out = chunk_gated_delta_rule_fwd(
        q, k, v, g, beta, scale=scale, cu_seqlens=cu_seqlens, output_final_state=True, transpose_state_layout=True,
        initial_state=state_pool if continue_from_pool else None,
        initial_state_indices=state_indices if continue_from_pool else None,
        final_state_out=state_pool, final_state_indices=state_indices, **forward_kwargs)
    return out[2], state_pool
