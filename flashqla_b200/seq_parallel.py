"""Cross-GPU sequence parallelism for the chunked forward and backward: ONE long sequence cut into contiguous
slices, one slice per rank, with a single all-gather of chunk-boundary states (forward) or of their gradients
(backward).

The reference has no multi-GPU path; the math is that of its intra-card context parallelism
(flash_qla/ops/gated_delta_rule/chunk/cp_context.py:117-176 and ``correct_initial_states``,
chunk/hopper/cp_fwd.py:253): the state at the end of a stretch of tokens is an affine function of the state
at its start, ``S_end = H + M @ S_start`` with ``H`` the end state reached from zero and ``M`` the K x K
transition matrix, and ``M`` is taken as zero once the accumulated decay of the stretch is below
``exp(-10)`` (cp.WARMUP_THRESHOLD).

Per rank:

1. chunk preparation of the slice (``g_cumsum``, ``A``, ``w``), the slice cut into local segments by the same
   planner as the single-GPU path (one segment if it does not cut);
2. the local warm-up / transition passes, chained from a ZERO incoming state, with one extra row that
   receives the end state of the last segment: ``H_slice``.  A second run of the chaining kernel on a buffer
   whose first row is the identity yields the prefix products of the transition matrices, the last of which
   is ``M_slice`` (all zero unless no segment of the slice decays below the threshold);
3. one ``all_gather`` of ``(H_slice, M_slice)``: ``2 * Hv * 64 KiB`` per rank;
4. every rank folds the summaries of the ranks before it into its incoming state, corrects its segment
   start states with the prefix products, and runs the main scan over its segments.

The final state of the sequence is the one the last rank computes.  Received data is ordinary local memory
(NCCL writes it there); no kernel of this library reads a peer's memory.

The backward mirrors this from the right: the gradient of the state at the START of a slice is an affine
function of the gradient at its end, ``dS_start = G + Md @ dS_end``; every rank computes ``(G, Md)`` of its slice
with one state-only launch of the reverse scan (zero start for ``G``, identity start and ``dO`` taken as zero
for ``Md``), one all-gather moves them, every rank folds the summaries of the ranks AFTER it into the gradient
entering its slice from the right and runs the ordinary backward on the slice.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, Optional, Tuple

import torch

from . import _cabi, cp
from .chunk import CHUNK, _launch_fwd, chunk_tables_workspace, new_w

_SP_PLANS: Dict[Tuple, "SpPlan"] = {}


@dataclass
class SpPlan:
    n_seg: int
    dev: Dict[str, torch.Tensor]
    tables: Dict[str, torch.Tensor]


def _sp_plan(tokens: int, num_v_heads: int, device: torch.device) -> SpPlan:
    """Local segments of a slice plus the extra export row behind the last one (device index arrays)."""
    key = (tokens, num_v_heads, str(device))
    plan = _SP_PLANS.get(key)
    if plan is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        base = cp.plan_segments([tokens], num_v_heads, sms)
        cu = base.cu if base.use_cp else [0, tokens]
        n_seg = len(cu) - 1
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
        plan = SpPlan(n_seg, dict(
            cu=i32(cu),
            # every segment has a successor row: the last one's is the export row n_seg
            seg_next=i32(list(range(1, n_seg + 1))),
            identity=i32(list(range(n_seg))),
            raw_first=i32([0, n_seg + 1]),
            # the main scan writes the state behind the last segment into row 0 of its final-state output
            seg_raw=i32([-1] * (n_seg - 1) + [0])), chunk_tables_workspace(cu, device))
        if len(_SP_PLANS) < 256:
            _SP_PLANS[key] = plan
    return plan


def fold_incoming_state(gathered: torch.Tensor, rank: int, initial_state: Optional[torch.Tensor]) -> torch.Tensor:
    """State entering the slice of ``rank``.  ``gathered`` is ``[world, 2, Hv, K, V]``: per rank the end state
    of its slice reached from zero and its transition matrix.  Pure torch, any device."""
    Hv, K, V = gathered.shape[2:]
    S = (torch.zeros(Hv, K, V, dtype=torch.float32, device=gathered.device) if initial_state is None
         else initial_state.reshape(Hv, K, V).to(torch.float32))
    for j in range(rank):
        S = gathered[j, 0] + torch.bmm(gathered[j, 1], S)
    return S


@dataclass
class _SliceContext:
    plan: SpPlan
    tensors: tuple
    scale: float
    cp_h0: torch.Tensor    # [n_seg + 1, Hv, 128, 128] segment start states for a zero incoming state
    prefix: torch.Tensor   # [n_seg + 1, Hv, 128, 128] prefix products of the transition matrices
    summary: torch.Tensor  # [2, Hv, 128, 128] = (H_slice, M_slice), what the all-gather sends


def slice_summary(q, k, v, g, beta, scale: Optional[float] = None) -> _SliceContext:
    """Steps 1 and 2 for the local slice ``q, k [1,T,Hk,128]``, ``v [1,T,Hv,128]``, ``g, beta [1,T,Hv]``."""
    if q.shape[0] != 1:
        raise ValueError(f"one sequence: the batch size is expected to be 1 rather than {q.shape[0]}")
    T, Hv = k.shape[1], beta.shape[2]
    if T % CHUNK != 0:
        raise ValueError(f"a slice must be a whole number of {CHUNK}-token chunks (the last rank included), got {T}")
    dev = k.device
    q, k, v, g, beta = (x if x.is_contiguous() else x.contiguous() for x in (q, k, v, g, beta))
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    plan = _sp_plan(T, Hv, dev)
    d, n_seg = plan.dev, plan.n_seg
    lib, stream = _cabi.lib(), _cabi.current_stream(dev)

    g_cumsum = torch.empty(1, T, Hv, dtype=torch.float32, device=dev)
    A = torch.empty(1, T, Hv, CHUNK, dtype=q.dtype, device=dev)
    w = new_w(k, beta)
    _launch_fwd(None, k, None, g, beta, None, None, g_cumsum, A, None, None, None, None, scale,
                flags=_cabi.CHUNK_PREPARE_ONLY, w=w)

    warm_limit = torch.empty(n_seg, Hv, dtype=torch.int32, device=dev)
    m_limit = torch.empty(n_seg, Hv, dtype=torch.int32, device=dev)
    pa = _cabi.QlaCpPlanArgs(num_segments=n_seg, num_v_heads=Hv, threshold=cp.WARMUP_THRESHOLD,
                             g_cumsum=g_cumsum.data_ptr(), cu_seqlens=d["cu"].data_ptr(),
                             seg_next=d["seg_next"].data_ptr(), warm_limit=warm_limit.data_ptr(),
                             m_limit=m_limit.data_ptr())
    with torch.cuda.device(dev):
        _cabi.check(lib.qla_cp_plan(pa, stream), "qla_cp_plan")

    cp_h0 = torch.zeros(n_seg + 1, Hv, 128, 128, dtype=torch.float32, device=dev)
    flags = _cabi.CHUNK_STATE_ONLY | _cabi.CHUNK_SKIP_PREPARE
    M = torch.empty(n_seg, Hv, 128, 128, dtype=torch.float32, device=dev)
    # warm-up pass and transition-matrix pass as one launch
    _launch_fwd(None, k, v, None, beta, None, d["cu"], g_cumsum, A, None, None, None, cp_h0, scale, flags=flags,
                seq_map=d["seg_next"], chunk_limit=warm_limit, num_seqs=n_seg, w=w, tables=plan.tables,
                dual=(m_limit, d["identity"], M))
    prefix = torch.zeros(n_seg + 1, Hv, 128, 128, dtype=torch.float32, device=dev)
    prefix[0] = torch.eye(128, dtype=torch.float32, device=dev)
    for buf in (cp_h0, prefix):
        ca = _cabi.QlaCpChainArgs(num_raw_seqs=1, num_v_heads=Hv, h0=buf.data_ptr(), M=M.data_ptr(),
                                  m_limit=m_limit.data_ptr(), raw_first_seg=d["raw_first"].data_ptr())
        with torch.cuda.device(dev):
            _cabi.check(lib.qla_cp_chain(ca, stream), "qla_cp_chain")
    summary = torch.stack((cp_h0[n_seg], prefix[n_seg]))
    return _SliceContext(plan, (q, k, v, beta, g_cumsum, A, w, M, m_limit), scale, cp_h0, prefix, summary)


def slice_forward(ctx: _SliceContext, incoming: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Step 4 for the local slice: ``incoming`` ``[Hv,128,128]`` is the state entering it (``None`` = zero).
    Returns ``(o, state behind the slice)``."""
    q, k, v, beta, g_cumsum, A, w, _, _ = ctx.tensors
    plan, n_seg = ctx.plan, ctx.plan.n_seg
    start = ctx.cp_h0[:n_seg]
    if incoming is not None:
        # start state of segment s = its start for a zero incoming state + (M_{s-1} ... M_0) @ incoming
        start = start + torch.matmul(ctx.prefix[:n_seg], incoming.to(torch.float32).unsqueeze(0))
    start = start.contiguous()
    o = torch.empty_like(v)
    end_state = torch.empty(1, v.shape[2], 128, 128, dtype=torch.float32, device=v.device)
    _launch_fwd(q, k, v, None, beta, start, plan.dev["cu"], g_cumsum, A, o, None, None, end_state, ctx.scale,
                flags=_cabi.CHUNK_SKIP_PREPARE, seq_map=plan.dev["seg_raw"], num_seqs=n_seg, w=w,
                tables=plan.tables)
    return o, end_state


def chunk_gated_delta_rule_fwd_sp(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    group=None,
    broadcast_final_state: bool = False,
    gather: Optional[Callable[[torch.Tensor], torch.Tensor]] = None,
    return_incoming_state: bool = False,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Forward of one sequence whose tokens are spread over the ranks of ``group`` in rank order; every rank
    passes ITS slice (``[1, T_rank, ...]``, a whole number of 64-token chunks; slices may differ in length)
    and gets ``o`` of its slice.  ``initial_state`` ``[1,Hv,128,128]`` is the state before the first token
    of the sequence (read on every rank that passes it; only its value on rank 0's side of the fold matters,
    so pass the same tensor everywhere or ``None``).  The final state is returned on the last rank (on every
    rank with ``broadcast_final_state``), ``None`` elsewhere.  One collective: an all-gather of
    ``2 * Hv * 64 KiB`` per rank.  ``gather`` replaces the collective (a callable from the local summary to
    the ``[world, 2, Hv, 128, 128]`` stack) for callers that move the summaries themselves.  With
    ``return_incoming_state`` a third value is returned: the state entering this rank's slice ``[1,Hv,128,128]``
    (``None`` when it is zero), which ``chunk_gated_delta_rule_bwd_sp`` takes."""
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ctx = slice_summary(q, k, v, g, beta, scale)
    if gather is not None:
        gathered = gather(ctx.summary)
    else:
        gathered = torch.empty((world,) + tuple(ctx.summary.shape), dtype=torch.float32, device=q.device)
        dist.all_gather_into_tensor(gathered, ctx.summary.contiguous(), group=group)
    incoming = None
    if rank > 0 or initial_state is not None:
        incoming = fold_incoming_state(gathered, rank, initial_state)
    o, end_state = slice_forward(ctx, incoming)
    extra = ((incoming.unsqueeze(0) if incoming is not None else None),) if return_incoming_state else ()
    if broadcast_final_state:
        dist.broadcast(end_state, src=dist.get_global_rank(group, world - 1) if group is not None else world - 1,
                       group=group)
        return (o, end_state) + extra
    return (o, (end_state if rank == world - 1 else None)) + extra


# ------------------------------------------------------------------------------------------------ backward

def fold_incoming_gradient(gathered: torch.Tensor, rank: int, dht: Optional[torch.Tensor]) -> torch.Tensor:
    """Gradient of the state BEHIND the slice of ``rank`` (what enters its reverse scan).  ``gathered`` is
    ``[world, 2, Hv, K, V]``: per rank ``G`` (the start-state gradient of its slice for a zero gradient behind
    it) and ``Md``.  ``dht`` is the gradient of the sequence's final state.  Pure torch, any device."""
    world = gathered.shape[0]
    Hv, K, V = gathered.shape[2:]
    D = (torch.zeros(Hv, K, V, dtype=torch.float32, device=gathered.device) if dht is None
         else dht.reshape(Hv, K, V).to(torch.float32))
    for j in range(world - 1, rank, -1):
        D = gathered[j, 0] + torch.bmm(gathered[j, 1], D)
    return D


@dataclass
class _SliceBackwardContext:
    tensors: tuple          # q, k, v, beta, do, g_cumsum, A, h, v_new, w, incoming
    scale: float
    summary: torch.Tensor   # [2, Hv, 128, 128] = (G_slice, Md_slice)


def slice_backward_summary(q, k, v, g, beta, do, incoming: Optional[torch.Tensor] = None,
                           scale: Optional[float] = None) -> _SliceBackwardContext:
    """Forward recomputation of the slice from the state entering it (``g_cumsum``, ``A``, ``w``, ``h``,
    ``v_new``) and the slice's ``(G, Md)``: ONE launch of the reverse scan, state-only, its two halves starting
    from zero and from the identity."""
    from .chunk import chunk_gated_delta_rule_fwd
    from .utils import device_status
    if q.shape[0] != 1:
        raise ValueError(f"one sequence: the batch size is expected to be 1 rather than {q.shape[0]}")
    T, Hk, Hv = k.shape[1], k.shape[2], beta.shape[2]
    if T % CHUNK != 0:
        raise ValueError(f"a slice must be a whole number of {CHUNK}-token chunks (the last rank included), got {T}")
    dev = k.device
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    q, k, v, beta, do = (x if x.is_contiguous() else x.contiguous() for x in (q, k, v, beta, do))
    if do.dtype != q.dtype:
        do = do.to(q.dtype)
    g_cumsum, A, _, h, _, v_new, w = chunk_gated_delta_rule_fwd(
        q, k, v, g, beta, scale=scale, initial_state=incoming, output_h=True, output_v_new=True, output_w=True)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev)
    n_chunks = T // CHUNK
    summary = torch.empty(2, 1, Hv, 128, 128, dtype=torch.float32, device=dev)
    limit = torch.full((1, Hv), n_chunks, dtype=torch.int32, device=dev)
    cu, row0 = i32([0, T]), i32([0])
    sa = _cabi.QlaChunkBwdArgs(
        batch=1, seq_len=T, num_seqs=1, num_k_heads=Hk, num_v_heads=Hv, qkv_dtype=_cabi.dtype_code(q.dtype),
        beta_dtype=_cabi.QLA_DT_F32, flags=_cabi.CHUNK_STATE_ONLY | _cabi.CHUNK_DUAL_TRANSITION, scale=scale,
        q=_cabi.ptr(q), k=_cabi.ptr(k), g_cumsum=_cabi.ptr(g_cumsum), w=_cabi.ptr(w), d_o=_cabi.ptr(do),
        cu_seqlens=cu.data_ptr(), dh0=summary[0].data_ptr(), status=_cabi.ptr(device_status(dev)),
        chunk_limit=limit.data_ptr(), out_map=row0.data_ptr(), chunk_limit_b=limit.data_ptr(),
        out_map_b=row0.data_ptr(), out_b=summary[1].data_ptr())
    with torch.cuda.device(dev):
        _cabi.check(_cabi.lib().qla_chunk_bwd(sa, _cabi.current_stream(dev)), "qla_chunk_bwd (state-only)")
    return _SliceBackwardContext((q, k, v, beta, do, g_cumsum, A, h, v_new, w, incoming), scale, summary[:, 0])


def slice_backward(ctx: _SliceBackwardContext, incoming_gradient: Optional[torch.Tensor]):
    """The ordinary backward on the slice with ``incoming_gradient`` ``[Hv,128,128]`` entering from the right
    (``None`` = zero).  Returns ``(dq, dk, dv, dbeta, dg, dS_start)``; ``dS_start`` is the gradient of the state
    entering the slice: on the first rank that of the sequence's initial state."""
    from .chunk import chunk_gated_delta_rule_bwd
    q, k, v, beta, do, g_cumsum, A, h, v_new, w, incoming = ctx.tensors
    Hv = beta.shape[2]
    h0 = incoming if incoming is not None else torch.zeros(1, Hv, 128, 128, dtype=torch.float32, device=q.device)
    dht = incoming_gradient.unsqueeze(0).contiguous() if incoming_gradient is not None else None
    return chunk_gated_delta_rule_bwd(q, k, v, g_cumsum, beta, A, do, dht=dht, scale=ctx.scale, initial_state=h0,
                                      h=h, v_new=v_new, w=w)


def chunk_gated_delta_rule_bwd_sp(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    do: torch.Tensor,
    incoming_state: Optional[torch.Tensor] = None,
    dht: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    group=None,
    gather: Optional[Callable[[torch.Tensor], torch.Tensor]] = None,
):
    """Backward of ``chunk_gated_delta_rule_fwd_sp``: every rank passes its slice of the inputs (``g`` the raw
    gates), ``do`` of its slice and the state that entered its slice in the forward (``incoming_state``, the third
    value of the forward with ``return_incoming_state``); ``dht`` ``[1,Hv,128,128]`` is the gradient of the
    sequence's final state (same tensor on every rank, or ``None``).  Returns ``(dq, dk, dv, dbeta, dg, dS_start)``
    of the slice.  One collective: an all-gather of ``2 * Hv * 64 KiB`` per rank."""
    import torch.distributed as dist
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ctx = slice_backward_summary(q, k, v, g, beta, do, incoming_state, scale)
    if gather is not None:
        gathered = gather(ctx.summary)
    else:
        gathered = torch.empty((world,) + tuple(ctx.summary.shape), dtype=torch.float32, device=q.device)
        dist.all_gather_into_tensor(gathered, ctx.summary.contiguous(), group=group)
    incoming_gradient = None
    if rank < world - 1 or dht is not None:
        incoming_gradient = fold_incoming_gradient(gathered, rank, dht)
    return slice_backward(ctx, incoming_gradient)
