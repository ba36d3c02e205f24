"""Recurrent GDN update: decode, spec-decode verify, tree verify, ragged sequences.

Host-side mirror of ``fused_sigmoid_gating_delta_rule_update``
(reference: flash_qla/ops/gated_delta_rule/recurrent_fused.py:6287-7537): same name, argument
order, defaults and error behaviour; the work is one launch of ``qla_recurrent_update`` in the
C-ABI library.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _cabi
from .utils import device_status


def _state_view(state: torch.Tensor, Hv: int, K: int, V: int) -> torch.Tensor:
    # reference: _contiguous_state_view, recurrent_fused.py:6270-6284.  The pool is updated in
    # place, so a non-contiguous pool (which the reference would silently copy, losing the update)
    # is rejected.
    if state.dim() != 4:
        raise ValueError("initial_state_source must be a 4-D tensor")
    if state.shape[1] != Hv:
        raise ValueError(f"initial_state_source head dim {state.shape[1]} != num_value_heads {Hv}")
    if tuple(state.shape[2:]) not in ((V, K), (K, V)):
        raise ValueError("initial_state_source must have trailing shape [V, K] for recurrent GDN layout "
                         "or [K, V] when K == V-compatible contiguous storage is intended")
    if not state.is_contiguous():
        raise ValueError("initial_state_source must be contiguous: it is updated in place")
    return state


def _i32(t: Optional[torch.Tensor], device) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t.to(device=device, dtype=torch.int32).contiguous()


def fused_sigmoid_gating_delta_rule_update(
    A_log: torch.Tensor,
    a: torch.Tensor,
    dt_bias: torch.Tensor,
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    b: torch.Tensor,
    initial_state_source: torch.Tensor,
    initial_state_indices: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    softplus_beta: float = 1.0,
    softplus_threshold: float = 20.0,
    use_qk_l2norm_in_kernel: bool = True,
    cu_seqlens: Optional[torch.Tensor] = None,
    disable_state_update: bool = False,
    intermediate_states_buffer: Optional[torch.Tensor] = None,
    intermediate_state_indices: Optional[torch.Tensor] = None,
    cache_steps: Optional[int] = None,
    retrieve_parent_token: Optional[torch.Tensor] = None,
    block_dv: Optional[int] = None,
    assume_regular: bool = False,
    b_is_beta: bool = False,
    a_is_log_decay: bool = False,
) -> torch.Tensor:
    """One GDN step per token, state ``[slots, Hv, V, K]`` (fp32, or bf16 as an addition to the reference)
    updated in place; returns ``o``.  Out-of-range slots, parents or cu_seqlens boundaries never touch memory and
    are reported through ``check_device_status()``.

    ``g = a`` if ``a_is_log_decay`` else ``-exp(A_log) * softplus(a + dt_bias)``; ``beta = b`` if
    ``b_is_beta`` else ``sigmoid(b)``.  Unlike the reference, both flags are honoured on every
    path (the reference drops them outside single-token decode, recurrent_fused.py:7364-7393).
    ``block_dv`` is accepted for compatibility; values <= 16 select the 16-row tile.
    """
    if q.shape[0] != 1 or k.shape[0] != 1 or v.shape[0] != 1:
        raise ValueError("FlashQLA recurrent GDN kernel expects flattened [1, total_tokens, ...] inputs")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("q, k, and v must have the same dtype")
    if not q.is_cuda:
        raise ValueError("FlashQLA recurrent GDN kernel requires CUDA tensors")
    q, k, v, a, b = (x if x.is_contiguous() else x.contiguous() for x in (q, k, v, a, b))

    _, NT, Hk, K = q.shape
    _, _, Hv, V = v.shape
    if Hv % Hk != 0:
        raise ValueError("num_value_heads must be divisible by num_key_heads")
    if K != 128 or V != 128:
        raise ValueError("FlashQLA recurrent GDN kernel currently specializes Qwen GDN K=V=128")
    if tuple(a.shape) != (1, NT, Hv):
        raise ValueError(f"a shape {tuple(a.shape)} does not match [1, total_tokens, HV]")
    if tuple(b.shape) != (1, NT, Hv):
        raise ValueError(f"b shape {tuple(b.shape)} does not match [1, total_tokens, HV]")
    if a.dtype != b.dtype:
        b = b.to(a.dtype)
    if not a_is_log_decay:
        if tuple(A_log.shape) != (Hv,):
            raise ValueError("A_log must have shape [HV]")
        if tuple(dt_bias.shape) != (Hv,):
            raise ValueError("dt_bias must have shape [HV]")
        A_log, dt_bias = A_log.contiguous(), dt_bias.contiguous()

    state = _state_view(initial_state_source, Hv, K, V)
    if state.dtype not in (torch.float32, torch.bfloat16):
        # the reference's pools are float32 (recurrent_fused.py:6292); bfloat16 pools are an addition
        raise NotImplementedError("initial_state_source must be float32 or bfloat16")
    dev = q.device
    cu = _i32(cu_seqlens, dev)
    sidx = _i32(initial_state_indices, dev)
    if cu is not None:
        N = cu.numel() - 1
    elif sidx is not None:
        N = sidx.numel()
    else:
        N = state.shape[0]
    if sidx is not None and sidx.numel() != N:
        raise ValueError("initial_state_indices length must equal num_sequences")
    if sidx is None and N > state.shape[0]:
        raise ValueError("cu_seqlens length must equal num_sequences + 1")
    tokens_per_seq = 0
    if cu is None or assume_regular:
        if N == 0 or NT % N != 0:
            if assume_regular:
                raise ValueError("assume_regular=True requires total_tokens divisible by num_sequences")
            raise ValueError("total_tokens must be divisible by num_sequences when cu_seqlens is omitted")
        tokens_per_seq = NT // N
        cu = None
    if scale is None:
        scale = K ** -0.5

    inter = intermediate_states_buffer
    cidx = None
    inter_steps = 0
    if inter is not None:
        if inter.dim() != 5 or inter.shape[2] != Hv or tuple(inter.shape[3:]) not in ((V, K), (K, V)):
            raise ValueError("intermediate_states_buffer must be [slots, steps, HV, V, K]")
        if not inter.is_contiguous():
            raise ValueError("intermediate_states_buffer must be contiguous: it is written in place")
        if inter.dtype not in (torch.float32, torch.bfloat16):
            raise NotImplementedError("intermediate_states_buffer must be float32 or bfloat16")
        inter_steps = inter.shape[1]
        if cache_steps is None:
            cache_steps = inter_steps
        if inter_steps < cache_steps:
            raise ValueError("intermediate_states_buffer cache dimension is smaller than cache_steps")
        cidx = _i32(intermediate_state_indices, dev)
        if cidx is None and inter.shape[0] < N:
            raise ValueError("intermediate_states_buffer must have at least num_sequences slots")
        if tokens_per_seq > inter_steps:
            raise ValueError("intermediate_states_buffer cache dimension is smaller than tokens per sequence")
    parents = _i32(retrieve_parent_token, dev)
    if parents is not None:
        if inter is None:
            raise ValueError("retrieve_parent_token requires intermediate_states_buffer")
        if parents.dim() != 2 or parents.shape[0] != N:
            raise ValueError("retrieve_parent_token first dimension must equal num_sequences")
        if tokens_per_seq > parents.shape[1]:
            raise ValueError("retrieve_parent_token has fewer columns than tokens per sequence")

    o = torch.empty_like(v)
    flags = ((_cabi.REC_QK_L2NORM if use_qk_l2norm_in_kernel else 0)
             | (_cabi.REC_DISABLE_STATE_UPDATE if disable_state_update else 0)
             | (_cabi.REC_A_IS_LOG_DECAY if a_is_log_decay else 0)
             | (_cabi.REC_B_IS_BETA if b_is_beta else 0))
    rows = 0 if block_dv is None else (16 if block_dv <= 16 else 32)
    args = _cabi.QlaRecurrentArgs(
        num_seqs=N, total_tokens=NT, tokens_per_seq=tokens_per_seq, num_k_heads=Hk, num_v_heads=Hv,
        qkv_dtype=_cabi.dtype_code(q.dtype), a_dtype=_cabi.dtype_code(a.dtype),
        a_log_dtype=0 if a_is_log_decay else _cabi.dtype_code(A_log.dtype),
        dt_bias_dtype=0 if a_is_log_decay else _cabi.dtype_code(dt_bias.dtype),
        inter_dtype=0 if inter is None else _cabi.dtype_code(inter.dtype),
        inter_steps=inter_steps, parents_stride=0 if parents is None else parents.stride(0),
        flags=flags, rows_per_cta=rows, state_slots=state.shape[0],
        inter_slots=0 if inter is None else inter.shape[0],
        scale=float(scale), softplus_beta=float(softplus_beta),
        softplus_threshold=float(softplus_threshold),
        A_log=None if a_is_log_decay else _cabi.ptr(A_log), a=_cabi.ptr(a),
        dt_bias=None if a_is_log_decay else _cabi.ptr(dt_bias),
        q=_cabi.ptr(q), k=_cabi.ptr(k), v=_cabi.ptr(v), b=_cabi.ptr(b), state=_cabi.ptr(state),
        state_indices=_cabi.ptr(sidx), cu_seqlens=_cabi.ptr(cu), inter=_cabi.ptr(inter),
        inter_indices=_cabi.ptr(cidx), parents=_cabi.ptr(parents), o=_cabi.ptr(o),
        status=_cabi.ptr(device_status(dev)), state_dtype=_cabi.dtype_code(state.dtype),
        parents_steps=0 if parents is None else parents.shape[1])
    with torch.cuda.device(dev):
        code = _cabi.lib().qla_recurrent_update(args, _cabi.current_stream(dev))
    _cabi.check(code, "qla_recurrent_update")
    return o


flashqla_recurrent_gdn_update = fused_sigmoid_gating_delta_rule_update


def commit_verified_state(
    initial_state_source: torch.Tensor,
    intermediate_states_buffer: torch.Tensor,
    num_accepted: torch.Tensor,
    initial_state_indices: Optional[torch.Tensor] = None,
    intermediate_state_indices: Optional[torch.Tensor] = None,
) -> None:
    """After a verify step (``disable_state_update=True`` with ``intermediate_states_buffer``): write the state
    that follows the last ACCEPTED draft token of every sequence back into the pool, in place,
    ``state[initial_state_indices[n]] = intermediate[intermediate_state_indices[n], num_accepted[n] - 1]``;
    ``num_accepted[n] == 0`` leaves a sequence's state as it was.  Argument names follow
    ``fused_sigmoid_gating_delta_rule_update``; the reference leaves this step to its caller."""
    state, inter = initial_state_source, intermediate_states_buffer
    if inter.dim() != 5 or tuple(inter.shape[3:]) != (128, 128):
        raise ValueError("intermediate_states_buffer must be [slots, steps, HV, 128, 128]")
    Hv = inter.shape[2]
    if not state.is_contiguous() or not inter.is_contiguous():
        raise ValueError("the state pool and intermediate_states_buffer must be contiguous")
    if state.dtype not in (torch.float32, torch.bfloat16) or state.numel() % (Hv * 128 * 128) != 0:
        raise ValueError("initial_state_source must be a float32 or bfloat16 pool of [HV, 128, 128] states")
    if inter.dtype not in (torch.float32, torch.bfloat16):
        raise NotImplementedError("intermediate_states_buffer must be float32 or bfloat16")
    dev = state.device
    acc = _i32(num_accepted, dev)
    sidx = _i32(initial_state_indices, dev)
    cidx = _i32(intermediate_state_indices, dev)
    args = _cabi.QlaStateCommitArgs(
        num_seqs=acc.numel(), num_v_heads=Hv, inter_dtype=_cabi.dtype_code(inter.dtype), inter_steps=inter.shape[1],
        inter_slots=inter.shape[0], state_slots=state.numel() // (Hv * 128 * 128), inter=_cabi.ptr(inter),
        accepted=_cabi.ptr(acc), state_indices=_cabi.ptr(sidx), inter_indices=_cabi.ptr(cidx),
        state=_cabi.ptr(state), status=_cabi.ptr(device_status(dev)), state_dtype=_cabi.dtype_code(state.dtype))
    with torch.cuda.device(dev):
        code = _cabi.lib().qla_state_commit(args, _cabi.current_stream(dev))
    _cabi.check(code, "qla_state_commit")
