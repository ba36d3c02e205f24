"""Chunked prefill / training op: host-side mirror of the reference's chunk API.

Reference: flash_qla/ops/gated_delta_rule/chunk/__init__.py - ``chunk_gated_delta_rule_fwd`` (:23-86),
``chunk_gated_delta_rule_bwd`` (:89-182), ``ChunkGatedDeltaRuleFunction`` (:185-290) and
``chunk_gated_delta_rule`` (:294-350).  Same names, argument order, defaults and error behaviour;
the work happens in the C-ABI library (``qla_chunk_fwd`` ...).
"""
from __future__ import annotations

from typing import Optional

import torch

from . import _cabi, cp
from .utils import device_status, host_seqlens, l2norm, longest_first_order

CHUNK = 64


def _check_common(q, k, v, g, beta, initial_state, cu_seqlens, transpose_state_layout):
    assert q.dtype == k.dtype == v.dtype, "q, k, v must share a dtype"
    assert q.dtype != torch.float32, "ChunkGatedDeltaRuleFunction does not support float32. Please use bfloat16."
    assert q.dim() == 4 and k.shape == q.shape and v.dim() == 4, "q,k [B,T,Hk,K]; v [B,T,Hv,V]"
    B, T, Hk, K = q.shape
    Hv, V = v.shape[2], v.shape[3]
    assert K == 128 and V == 128, "K = V = 128 only"
    assert Hv % Hk == 0, "the number of v heads must be a multiple of the number of q/k heads"
    assert tuple(g.shape) == (B, T, Hv) and tuple(beta.shape) == (B, T, Hv), "g, beta must be [B,T,Hv]"
    N = B
    if cu_seqlens is not None:
        if B != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {B} when using `cu_seqlens`."
                "Please flatten variable-length inputs before processing.")
        N = cu_seqlens.numel() - 1
    if initial_state is not None:
        if initial_state.shape[0] != N:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {N} rather than {initial_state.shape[0]}.")
        want = (N, Hv, V, K) if transpose_state_layout else (N, Hv, K, V)
        if tuple(initial_state.shape) != want:
            raise ValueError(f"initial_state must have shape {want}, got {tuple(initial_state.shape)}")
    return B, T, Hk, Hv, N


def _launch_fwd(q, k, v, g, beta, h0, cu, g_cumsum, A, o, h, v_new, final_state, scale, flags=0,
                seq_map=None, chunk_limit=None, num_seqs=None, w=None, tables=None, seq_order=None, rnorm=None,
                A_log=None, dt_bias=None, beta_out=None, h0_map=None, dual=None, out_norm=None, lead=None):
    """Fill ``QlaChunkFwdArgs`` from tensors and call ``qla_chunk_fwd`` on the current stream.  ``w`` is
    the per-chunk operand ``-(A diag(beta e^g) K)`` that the preparation step writes and the scan reads;
    it is allocated here when the call does both.  ``tables`` is an optional dict holding the ready-made
    chunk-table workspace of a fixed ``cu`` (``chunk_tables_workspace``: the segments of a context-parallel
    plan); calls that get it skip the table launch.  ``rnorm`` ``[B,T,Hk,2]`` switches the in-kernel q / k L2
    norm on: the preparation step writes the reciprocal row norms there, the scan reads them.  ``h0_map`` /
    ``seq_map`` are per-sequence rows of ``h0`` / ``final_state`` (state pools; ``-1`` = zero state / no output);
    the two share a dtype (fp32 or bf16).  ``dual = (chunk_limit_b, seq_map_b, final_state_b)`` adds the
    transition-matrix pass of context parallelism to a state-only launch.  ``lead`` ``[num_seqs, Hv]``: chunks in
    front of every interval that its scan runs first from a zero state (cp.segment_initial_states)."""
    dev = k.device
    if w is None:
        assert not flags & _cabi.CHUNK_SKIP_PREPARE, "a scan without preparation needs the prepared w"
        w = new_w(k, beta)
    B, T, Hk = k.shape[0], k.shape[1], k.shape[2]
    Hv = beta.shape[2]
    if cu is not None:  # packed view: [B, T, ...] is contiguous, i.e. [1, B*T, ...]
        B, T = 1, B * T
    N = num_seqs if num_seqs is not None else (cu.numel() - 1 if cu is not None else B)
    status = device_status(dev)
    if rnorm is not None:
        flags |= _cabi.CHUNK_QK_L2NORM
    if A_log is not None:
        flags |= _cabi.CHUNK_GATE_ACT
    if beta_out is not None:
        flags |= _cabi.CHUNK_BETA_LOGIT
    state_dtype = torch.float32
    for st in (final_state, h0 if not flags & _cabi.CHUNK_H0_KV_F32 else None):
        if st is not None:
            state_dtype = st.dtype
    dual_args = {}
    if out_norm is not None:  # (gate z, weight, eps): the gated RMS norm behind the op as an epilogue of the scan
        flags |= _cabi.CHUNK_OUT_GATED_RMSNORM
        dual_args.update(norm_gate=_cabi.ptr(out_norm[0]), norm_weight=_cabi.ptr(out_norm[1]), norm_eps=float(out_norm[2]))
    if dual is not None:
        flags |= _cabi.CHUNK_DUAL_TRANSITION
        dual_args.update(chunk_limit_b=_cabi.ptr(dual[0]), seq_map_b=_cabi.ptr(dual[1]), final_state_b=_cabi.ptr(dual[2]))
    args = _cabi.QlaChunkFwdArgs(
        batch=B, seq_len=T, num_seqs=N, num_k_heads=Hk, num_v_heads=Hv,
        qkv_dtype=_cabi.dtype_code(k.dtype), gate_dtype=0 if g is None else _cabi.dtype_code(g.dtype),
        beta_dtype=_cabi.dtype_code(beta.dtype), flags=flags, max_chunks_per_seq=0, scale=float(scale),
        q=_cabi.ptr(q), k=_cabi.ptr(k), v=_cabi.ptr(v), g=_cabi.ptr(g), beta=_cabi.ptr(beta),
        h0=_cabi.ptr(h0), cu_seqlens=_cabi.ptr(cu), seq_map=_cabi.ptr(seq_map), seq_order=_cabi.ptr(seq_order),
        chunk_limit=_cabi.ptr(chunk_limit), g_cumsum=_cabi.ptr(g_cumsum), A=_cabi.ptr(A), w=_cabi.ptr(w), qk_rnorm=_cabi.ptr(rnorm),
        A_log=_cabi.ptr(A_log), dt_bias=_cabi.ptr(dt_bias), beta_out=_cabi.ptr(beta_out), o=_cabi.ptr(o),
        h=_cabi.ptr(h), v_new=_cabi.ptr(v_new), final_state=_cabi.ptr(final_state), workspace=None,
        workspace_bytes=0, status=_cabi.ptr(status), h0_map=_cabi.ptr(h0_map),
        state_dtype=_cabi.dtype_code(state_dtype), lead=_cabi.ptr(lead), **dual_args)
    lib = _cabi.lib()
    if tables is not None and "ws" in tables:
        ws = tables["ws"]
        args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
        args.flags = flags | _cabi.CHUNK_TABLES_READY
    else:
        ws_bytes = lib.qla_chunk_fwd_workspace_bytes(args)
        if ws_bytes:
            ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
            args.workspace, args.workspace_bytes = ws.data_ptr(), ws_bytes
    with torch.cuda.device(dev):
        code = lib.qla_chunk_fwd(args, _cabi.current_stream(dev))
    _cabi.check(code, "qla_chunk_fwd")


def chunk_tables_workspace(cu: list, device) -> dict:
    """The workspace ``qla_chunk_fwd`` keeps its chunk tables in, computed on the host for boundaries known
    there: ``[n + 1]`` int32 exclusive scans of ``ceil(len / 128)`` and of ``ceil(len / 64)``, each padded to
    16 bytes.  The upload is a blocking copy, so the tables are complete before any stream can use them."""
    n = len(cu) - 1
    padded = ((n + 1) * 4 + 15) // 16 * 4
    pair, chunk = [0], [0]
    for i in range(n):
        length = cu[i + 1] - cu[i]
        pair.append(pair[-1] + (length + 127) // 128)
        chunk.append(chunk[-1] + (length + CHUNK - 1) // CHUNK)
    host = torch.zeros(2 * padded, dtype=torch.int32)
    host[:n + 1] = torch.tensor(pair, dtype=torch.int32)
    host[padded:padded + n + 1] = torch.tensor(chunk, dtype=torch.int32)
    return {"ws": host.to(device).view(torch.uint8)}


def new_w(k, beta):
    """Uninitialised ``[B, T, Hv, 128]`` buffer for the operand ``w`` of ``_launch_fwd``."""
    return torch.empty(k.shape[0], k.shape[1], beta.shape[2], 128, dtype=k.dtype, device=k.device)


def rebuild_w(k, beta, g_cumsum, A, cu):
    """``w`` from a saved ``g_cumsum`` / ``A`` pair (one preparation launch, no scan)."""
    w = new_w(k, beta)
    _launch_fwd(None, k, None, None, beta, None, cu, g_cumsum, A, None, None, None, None, 1.0,
                flags=_cabi.CHUNK_PREPARE_ONLY | _cabi.CHUNK_A_GIVEN, w=w)
    return w


def launches_per_forward(varlen: bool, use_cp: bool = False) -> int:
    """Kernels of this library one forward call launches.  Plain: [chunk tables] + kkt_solve + chunk
    scan.  With context parallelism: [tables] + kkt_solve, plan (+ start states), warm-up / transition scan
    (one launch), chain, main scan (the chunk tables of the plan's segments are built on the host together
    with the plan)."""
    if use_cp:
        return (2 if varlen else 1) + 1 + 1 + 1 + 1
    return 3 if varlen else 2


def launches_per_backward(varlen: bool, use_cp: bool = False) -> int:
    """Kernels one backward call launches with h, v_new and w saved by the forward: [chunk tables] + reverse scan +
    per-chunk kernel; context parallelism adds the reverse plan, the state-only / transition scan (one launch), the
    reverse chain and the segments' chunk tables."""
    return (3 if varlen else 2) + (4 if use_cp else 0)


def make_scan_only(q, k, v, beta, g_cumsum, A, o, final_state, initial_state=None, cu_seqlens=None,
                   scale=None, auto_cp=True):
    """Return a callable that launches only the chunk scan (the dominant kernel) exactly as a forward
    call with these arguments would: over context-parallel segments when the planner chooses them
    (segment initial states are computed once, here), else over whole sequences.  ``g_cumsum`` and ``A``
    come from an earlier forward.  Used to time that kernel by itself."""
    dev = k.device
    B, T, Hv = k.shape[0], k.shape[1], beta.shape[2]
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    cu = None if cu_seqlens is None else cu_seqlens.to(device=dev, dtype=torch.int32).contiguous()
    lens = host_seqlens(cu_seqlens) if cu_seqlens is not None else [T] * B
    plan = cp.get_plan(lens, Hv, dev) if auto_cp else None
    w = rebuild_w(k, beta, g_cumsum, A, cu)
    if plan is not None and plan.use_cp:
        cp_h0, lead = cp.segment_initial_states(plan, k, v, beta, g_cumsum, A, w, initial_state, scale, _launch_fwd)

        def run():
            _launch_fwd(q, k, v, None, beta, cp_h0, plan.dev["cu"], g_cumsum, A, o, None, None, final_state,
                        scale, flags=_cabi.CHUNK_SKIP_PREPARE | _cabi.CHUNK_H0_KV_F32, seq_map=plan.dev["seg_raw"],
                        num_seqs=len(plan.seg_next), w=w, tables=plan.tables, lead=lead)
        return run

    def run():
        _launch_fwd(q, k, v, None, beta, initial_state, cu, g_cumsum, A, o, None, None, final_state, scale,
                    flags=_cabi.CHUNK_SKIP_PREPARE, w=w)
    return run


def forward_scan_only(q, k, v, beta, g_cumsum, A, o, final_state, initial_state=None, cu_seqlens=None,
                      scale=None):
    """Launch the chunk scan once over whole sequences (no context parallelism)."""
    make_scan_only(q, k, v, beta, g_cumsum, A, o, final_state, initial_state, cu_seqlens, scale,
                   auto_cp=False)()


def chunk_gated_delta_rule_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    output_final_state: bool = True,
    output_h: bool = False,
    auto_cp: bool = True,
    output_v_new: bool = False,
    transpose_state_layout: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    A_log: Optional[torch.Tensor] = None,
    dt_bias: Optional[torch.Tensor] = None,
    beta_is_logit: bool = False,
    output_w: bool = False,
    initial_state_indices: Optional[torch.Tensor] = None,
    final_state_out: Optional[torch.Tensor] = None,
    final_state_indices: Optional[torch.Tensor] = None,
    out_norm_gate: Optional[torch.Tensor] = None,
    out_norm_weight: Optional[torch.Tensor] = None,
    out_norm_eps: float = 1e-6,
):
    """Raw forward.  ``g`` is the per-token log decay; returns
    ``(g_cumsum, A, o, h | None, final_state | None[, v_new])`` where ``g_cumsum`` is the chunk-local
    cumulative gate and ``A`` the gated WY matrix ``[B,T,Hv,64]``, both in the form the backward
    expects.  ``use_qk_l2norm_in_kernel`` (an addition to the reference's raw forward): q and k are used as
    ``x * rsqrt(sum(x^2) + 1e-6)`` per row, with the factors folded into the kernels instead of a pass over q
    and k; ``A`` and ``h`` are then those of the normalised inputs.  Two more additions fold the layer's gate
    activations into the preparation kernel (the recurrent op always had them): with ``A_log`` / ``dt_bias``
    ``[Hv]`` the argument ``g`` is the raw gate input ``a`` and ``g = -exp(A_log) * softplus(a + dt_bias)``
    is used; with ``beta_is_logit`` the argument ``beta`` holds logits and ``sigmoid(beta)`` is used.  With
    ``output_w`` the prepared chunk operand ``w = -(A diag(beta e^g) K)`` ``[B,T,Hv,128]`` is appended to the
    result; the backward takes it back (``w=``) instead of rebuilding it from ``g_cumsum`` and ``A``.

    State pools (the slot-indexed initial states of the reference's recurrent op,
    recurrent_fused.py:6287-6311, for the chunked path): with ``initial_state_indices`` (int ``[N]``)
    ``initial_state`` is a pool ``[slots, Hv, ...]`` and sequence ``n`` starts from slot
    ``initial_state_indices[n]`` (``-1``: zero state); with ``final_state_out`` the final states are written
    into that tensor, sequence ``n`` into row ``final_state_indices[n]`` (``-1``: not written; no indices:
    row ``n``), and it is what the call returns as final state.  Pools may be fp32 or bf16 (both the same);
    the kernels index the slots themselves, nothing is gathered or scattered around the call.

    Output norm (the gated RMS norm that follows the op in a GDN layer): with ``out_norm_gate`` ``z``
    ``[B,T,Hv,128]`` (q/k/v dtype) and ``out_norm_weight`` ``[128]`` the returned ``o`` is
    ``o * rsqrt(mean(o^2, -1) + out_norm_eps) * weight * silu(z)``, applied to the output tile inside the scan
    (inference: not together with ``output_h`` / ``output_v_new``)."""
    B, T, Hk, Hv, N = _check_common(q, k, v, g, beta, None if initial_state_indices is not None else initial_state,
                                    cu_seqlens, transpose_state_layout)
    if (A_log is None) != (dt_bias is None):
        raise ValueError("A_log and dt_bias go together")
    dev = q.device
    if not q.is_cuda:
        raise ValueError("flashqla_b200 requires CUDA tensors")
    q, k, v, g, beta = (x if x.is_contiguous() else x.contiguous() for x in (q, k, v, g, beta))
    if scale is None:
        scale = q.shape[-1] ** -0.5
    pooled = initial_state_indices is not None or final_state_out is not None
    h0, h0_map, fs_map = None, None, None
    if initial_state is not None:
        if initial_state_indices is not None:
            if initial_state.dim() != 4 or initial_state.shape[1] != Hv or tuple(initial_state.shape[2:]) != (128, 128):
                raise ValueError(f"a state pool must be [slots, {Hv}, 128, 128], got {tuple(initial_state.shape)}")
            if initial_state.dtype not in (torch.float32, torch.bfloat16) or not initial_state.is_contiguous():
                raise ValueError("a state pool must be a contiguous float32 or bfloat16 tensor")
            if initial_state_indices.numel() != N:
                raise ValueError(f"initial_state_indices must have one entry per sequence ({N})")
            h0 = initial_state
            h0_map = initial_state_indices.to(device=dev, dtype=torch.int32).contiguous()
        else:
            h0 = initial_state if (pooled and initial_state.dtype == torch.bfloat16) else initial_state.to(torch.float32)
            h0 = h0 if h0.is_contiguous() else h0.contiguous()
    if final_state_out is not None:
        if final_state_out.dim() != 4 or final_state_out.shape[1] != Hv or tuple(final_state_out.shape[2:]) != (128, 128):
            raise ValueError(f"final_state_out must be [rows, {Hv}, 128, 128], got {tuple(final_state_out.shape)}")
        if final_state_out.dtype not in (torch.float32, torch.bfloat16) or not final_state_out.is_contiguous():
            raise ValueError("final_state_out must be a contiguous float32 or bfloat16 tensor")
        if h0 is not None and h0.dtype != final_state_out.dtype:
            raise ValueError("initial states and final_state_out must share a dtype")
        if final_state_indices is not None:
            if final_state_indices.numel() != N:
                raise ValueError(f"final_state_indices must have one entry per sequence ({N})")
            fs_map = final_state_indices.to(device=dev, dtype=torch.int32).contiguous()
        elif final_state_out.shape[0] < N:
            raise ValueError("final_state_out needs one row per sequence")
    elif final_state_indices is not None:
        raise ValueError("final_state_indices needs final_state_out")
    cu = None
    lens = None
    if cu_seqlens is not None:
        cu = cu_seqlens.to(device=dev, dtype=torch.int32).contiguous()
        lens = host_seqlens(cu_seqlens, total_tokens=B * T)

    g_cumsum = torch.empty(B, T, Hv, dtype=torch.float32, device=dev)
    A = torch.empty(B, T, Hv, CHUNK, dtype=q.dtype, device=dev)
    o = torch.empty_like(v)
    if lens is None:
        n_chunks = B * ((T + CHUNK - 1) // CHUNK)
        h_shape = (B, (T + CHUNK - 1) // CHUNK, Hv, 128, 128)
    else:
        n_chunks = sum((n + CHUNK - 1) // CHUNK for n in lens)
        h_shape = (1, n_chunks, Hv, 128, 128)
    h = torch.empty(h_shape, dtype=q.dtype, device=dev) if output_h else None
    v_new = torch.empty_like(v) if output_v_new else None
    rnorm = torch.empty(B, T, Hk, 2, dtype=torch.float32, device=dev) if use_qk_l2norm_in_kernel else None
    out_norm = None
    if out_norm_gate is not None:
        if out_norm_weight is None or tuple(out_norm_gate.shape) != tuple(v.shape) or out_norm_gate.dtype != v.dtype:
            raise ValueError("out_norm_gate must have v's shape and dtype and needs out_norm_weight [128]")
        if output_h or output_v_new:
            raise ValueError("the output norm is an inference epilogue: not with output_h / output_v_new")
        out_norm = (out_norm_gate.contiguous(), out_norm_weight.to(device=dev, dtype=torch.float32).contiguous(),
                    out_norm_eps)
    if final_state_out is not None:
        final_state = final_state_out
    else:
        fs_dtype = h0.dtype if (h0 is not None and pooled) else torch.float32
        final_state = torch.empty(N, Hv, 128, 128, dtype=fs_dtype, device=dev) if output_final_state else None
    act = {}
    if A_log is not None:
        act.update(A_log=A_log.to(device=dev, dtype=torch.float32).contiguous(),
                   dt_bias=dt_bias.to(device=dev, dtype=torch.float32).contiguous())
    beta_act = torch.empty(B, T, Hv, dtype=torch.float32, device=dev) if beta_is_logit else None
    if beta_act is not None:
        act.update(beta_out=beta_act)

    plan = cp.get_plan(lens if lens is not None else [T] * B, Hv, dev) if auto_cp else None
    w = new_w(k, beta)
    if plan is not None and plan.use_cp:
        # g_cumsum and A on the original sequences, then per-segment initial states, then the scan
        # over segments (segments are whole chunks, so chunk numbering is unchanged)
        _launch_fwd(q if rnorm is not None else None, k, None, g, beta, None, cu, g_cumsum, A, None, None, None, None,
                    scale, flags=_cabi.CHUNK_PREPARE_ONLY, w=w, rnorm=rnorm, **act)
        if beta_act is not None:
            beta = beta_act  # every later stage reads the activated values
        cp_h0, lead = cp.segment_initial_states(plan, k, v, beta, g_cumsum, A, w, h0, scale, _launch_fwd, rnorm=rnorm,
                                                h0_map=h0_map, h0_transposed=transpose_state_layout)
        seg_rows = plan.dev["seg_raw"]
        if fs_map is not None:  # segment -> sequence -> row of the caller's pool
            seg_rows = torch.where(seg_rows >= 0, fs_map[seg_rows.clamp(min=0).long()], seg_rows)
        _launch_fwd(q, k, v, None, beta, cp_h0, plan.dev["cu"], g_cumsum, A, o, h, v_new, final_state, scale,
                    flags=_cabi.CHUNK_SKIP_PREPARE | _cabi.CHUNK_H0_KV_F32 |
                    (_cabi.CHUNK_TRANSPOSE_STATE if transpose_state_layout else 0),
                    seq_map=seg_rows, num_seqs=len(plan.seg_next), w=w, tables=plan.tables, rnorm=rnorm,
                    out_norm=out_norm, lead=lead)
    else:
        # packed batches of unequal lengths: the longest sequences are handed to the GPU first
        order = longest_first_order(cu_seqlens, dev) if cu_seqlens is not None else None
        _launch_fwd(q, k, v, g, beta, h0, cu, g_cumsum, A, o, h, v_new, final_state, scale,
                    flags=_cabi.CHUNK_TRANSPOSE_STATE if transpose_state_layout else 0, seq_order=order, rnorm=rnorm,
                    w=w, h0_map=h0_map, seq_map=fs_map, out_norm=out_norm, **act)
    out = (g_cumsum, A, o, h, final_state)
    if output_v_new:
        out += (v_new,)
    if output_w:
        out += (w,)
    return out


def chunk_gated_delta_rule_bwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    A: torch.Tensor,
    do: torch.Tensor,
    dht: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    cu_seqlens: Optional[torch.Tensor] = None,
    h: Optional[torch.Tensor] = None,
    v_new: Optional[torch.Tensor] = None,
    transpose_state_layout: bool = False,
    w: Optional[torch.Tensor] = None,
    auto_cp: bool = True,
):
    """Raw backward.  ``g`` is the chunk-local cumulative gate and ``A`` the WY matrix returned by
    ``chunk_gated_delta_rule_fwd``; ``h`` / ``v_new`` / ``w`` are the forward's optional outputs: ``h`` and
    ``v_new`` are recomputed by a state-only scan when missing, ``w`` by one preparation launch.  Returns ``(dq, dk, dv, db, dg, dh0 | None)`` with
    ``dg`` w.r.t. the raw per-token gate and ``dh0`` present iff ``initial_state`` is given (the
    oracle's convention, tests/ref_gdr.py:378)."""
    B, T, Hk, Hv, N = _check_common(q, k, v, g, beta, initial_state, cu_seqlens, transpose_state_layout)
    dev = q.device
    q, k, v, beta, A, do = (x if x.is_contiguous() else x.contiguous() for x in (q, k, v, beta, A, do))
    g_cumsum = g.to(torch.float32)
    g_cumsum = g_cumsum if g_cumsum.is_contiguous() else g_cumsum.contiguous()
    if do.dtype != q.dtype:
        do = do.to(q.dtype)
    if scale is None:
        scale = q.shape[-1] ** -0.5
    h0 = None
    if initial_state is not None:
        h0 = initial_state.to(torch.float32).contiguous()
    if dht is not None:
        dht = dht.to(torch.float32).contiguous()
    cu = None
    lens = None
    if cu_seqlens is not None:
        cu = cu_seqlens.to(device=dev, dtype=torch.int32).contiguous()
        lens = host_seqlens(cu_seqlens, total_tokens=B * T)
    flags = _cabi.CHUNK_TRANSPOSE_STATE if transpose_state_layout else 0
    if h is None or v_new is None:
        n_chunks = B * ((T + CHUNK - 1) // CHUNK) if lens is None else sum((n + CHUNK - 1) // CHUNK for n in lens)
        h = torch.empty(n_chunks, Hv, 128, 128, dtype=q.dtype, device=dev)
        v_new = torch.empty_like(v)
        if w is None:  # the recomputation rebuilds w on its way: keep it
            w = new_w(k, beta)
            _launch_fwd(None, k, v, None, beta, h0, cu, g_cumsum, A, None, h, v_new, None, scale,
                        flags=flags | _cabi.CHUNK_STATE_ONLY | _cabi.CHUNK_A_GIVEN, w=w)
        else:
            _launch_fwd(None, k, v, None, beta, h0, cu, g_cumsum, A, None, h, v_new, None, scale,
                        flags=flags | _cabi.CHUNK_STATE_ONLY | _cabi.CHUNK_SKIP_PREPARE, w=w)
    if w is None:
        w = rebuild_w(k, beta, g_cumsum, A, cu)
    w = w if w.is_contiguous() else w.contiguous()
    h = h if h.is_contiguous() else h.contiguous()
    v_new = v_new if v_new.is_contiguous() else v_new.contiguous()

    dq = torch.empty_like(q)
    dk = torch.empty_like(k)
    dv = torch.empty_like(v)
    db = torch.empty(B, T, Hv, dtype=torch.float32, device=dev)
    dg = torch.empty(B, T, Hv, dtype=torch.float32, device=dev)
    dh0 = torch.empty(N, Hv, 128, 128, dtype=torch.float32, device=dev) if initial_state is not None else None
    Bk, Tk = (1, B * T) if cu is not None else (B, T)
    # Long sequences on few heads: the reverse scan is cut into the same segments as the forward's (cp.py)
    plan = cp.get_plan(lens if lens is not None else [T] * B, Hv, dev) if auto_cp else None
    seg = {}
    if plan is not None and plan.use_cp:
        seg_dht, seg_lead = cp.segment_end_gradients(plan, q, k, do, w, g_cumsum, dht, scale,
                                                     transposed=transpose_state_layout)
        seg = dict(num_segments=len(plan.seg_next), seg_cu=_cabi.ptr(plan.dev["cu"]), seg_dht=_cabi.ptr(seg_dht),
                   seg_dh0_map=_cabi.ptr(plan.dev["seg_start_of"]), seg_lead=_cabi.ptr(seg_lead))
    args = _cabi.QlaChunkBwdArgs(
        batch=Bk, seq_len=Tk, num_seqs=N, num_k_heads=Hk, num_v_heads=Hv, qkv_dtype=_cabi.dtype_code(q.dtype),
        beta_dtype=_cabi.dtype_code(beta.dtype), flags=flags, scale=float(scale),
        q=_cabi.ptr(q), k=_cabi.ptr(k), v=_cabi.ptr(v), g_cumsum=_cabi.ptr(g_cumsum), beta=_cabi.ptr(beta),
        A=_cabi.ptr(A), h=_cabi.ptr(h), v_new=_cabi.ptr(v_new), w=_cabi.ptr(w), d_o=_cabi.ptr(do), dht=_cabi.ptr(dht),
        cu_seqlens=_cabi.ptr(cu), dq=_cabi.ptr(dq), dk=_cabi.ptr(dk), dv=_cabi.ptr(dv), dbeta=_cabi.ptr(db),
        dg=_cabi.ptr(dg), dh0=_cabi.ptr(dh0), workspace=None, workspace_bytes=0,
        status=_cabi.ptr(device_status(dev)), **seg)
    lib = _cabi.lib()
    ws_bytes = lib.qla_chunk_bwd_workspace_bytes(args)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws_bytes
    with torch.cuda.device(dev):
        code = lib.qla_chunk_bwd(args, _cabi.current_stream(dev))
    _cabi.check(code, "qla_chunk_bwd")
    return dq, dk, dv, db, dg, dh0


class ChunkGatedDeltaRuleFunction(torch.autograd.Function):
    """Autograd wrapper (reference: chunk/__init__.py:185-290).  The forward keeps ``h``, ``v_new`` and the
    prepared operand ``w`` so that the backward does not have to recompute them."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens,
                transpose_state_layout, keep_for_backward=True):
        # h and v_new are only kept when a backward can follow.  needs_input_grad reflects requires_grad of the
        # inputs even under torch.no_grad(), and grad mode is always off inside forward(), so the caller
        # passes whether gradients were enabled at the call.
        need_grad = keep_for_backward and any(ctx.needs_input_grad)
        out = chunk_gated_delta_rule_fwd(
            q, k, v, g, beta, scale=scale, initial_state=initial_state, cu_seqlens=cu_seqlens,
            output_final_state=output_final_state, output_h=need_grad, output_v_new=need_grad,
            transpose_state_layout=transpose_state_layout, output_w=need_grad)
        g_cumsum, A, o, h, final_state = out[:5]
        v_new, w = (out[5], out[6]) if need_grad else (None, None)
        ctx.save_for_backward(q, k, v, g_cumsum, beta, A, initial_state, cu_seqlens, h, v_new, w)
        ctx.scale = scale
        ctx.transpose_state_layout = transpose_state_layout
        ctx.g_dtype, ctx.beta_dtype = g.dtype, beta.dtype
        return o.to(q.dtype), final_state

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, do, dht):
        q, k, v, g_cumsum, beta, A, initial_state, cu_seqlens, h, v_new, w = ctx.saved_tensors
        dq, dk, dv, db, dg, dh0 = chunk_gated_delta_rule_bwd(
            q, k, v, g_cumsum, beta, A, do, dht=dht, scale=ctx.scale, initial_state=initial_state,
            cu_seqlens=cu_seqlens, h=h, v_new=v_new, transpose_state_layout=ctx.transpose_state_layout, w=w)
        if dh0 is not None and initial_state is not None:
            dh0 = dh0.to(initial_state.dtype)
        return (dq, dk, dv, dg.to(ctx.g_dtype), db.to(ctx.beta_dtype), None, dh0, None, None, None, None)


class ChunkGatedDeltaRuleFusedFunction(torch.autograd.Function):
    """Autograd wrapper of the forward with the layer's prologue folded into the kernels (q / k L2 norm, gate
    activation ``g = -exp(A_log) softplus(a + dt_bias)``, ``beta = sigmoid(b)``).  The forward runs the fused
    kernels (no elementwise pass over q, k, a, b); the backward re-forms the normalised / activated inputs with
    elementwise torch operations, runs the chunk backward on them and applies the chain rule of the three
    prologue maps to what comes back.  The reference applies these maps as separate differentiable passes in
    front of its op (chunk/__init__.py:332-334 for the L2 norm)."""

    @staticmethod
    @torch.amp.custom_fwd(device_type="cuda")
    def forward(ctx, q, k, v, g, beta, A_log, dt_bias, scale, initial_state, output_final_state, cu_seqlens,
                transpose_state_layout, use_l2norm, use_gate, use_beta_sigmoid):
        out = chunk_gated_delta_rule_fwd(
            q, k, v, g, beta, scale=scale, initial_state=initial_state, cu_seqlens=cu_seqlens,
            output_final_state=output_final_state, output_h=True, output_v_new=True, output_w=True,
            transpose_state_layout=transpose_state_layout, use_qk_l2norm_in_kernel=use_l2norm,
            A_log=A_log if use_gate else None, dt_bias=dt_bias if use_gate else None, beta_is_logit=use_beta_sigmoid)
        g_cumsum, A, o, h, final_state, v_new, w = out
        ctx.save_for_backward(q, k, v, g, beta, A_log, dt_bias, g_cumsum, A, initial_state, cu_seqlens, h, v_new, w)
        ctx.scale, ctx.transpose_state_layout = scale, transpose_state_layout
        ctx.flags = (use_l2norm, use_gate, use_beta_sigmoid)
        return o.to(q.dtype), final_state

    @staticmethod
    @torch.amp.custom_bwd(device_type="cuda")
    def backward(ctx, do, dht):
        q, k, v, g_in, beta_in, A_log, dt_bias, g_cumsum, A, initial_state, cu_seqlens, h, v_new, w = ctx.saved_tensors
        use_l2norm, use_gate, use_beta_sigmoid = ctx.flags
        qn, kn = (l2norm(q), l2norm(k)) if use_l2norm else (q, k)
        beta = torch.sigmoid(beta_in.float()) if use_beta_sigmoid else beta_in
        dq, dk, dv, db, dg, dh0 = chunk_gated_delta_rule_bwd(
            qn, kn, v, g_cumsum, beta, A, do, dht=dht, scale=ctx.scale, initial_state=initial_state,
            cu_seqlens=cu_seqlens, h=h, v_new=v_new, transpose_state_layout=ctx.transpose_state_layout, w=w)
        if use_l2norm:
            # x_hat = x r with r = (sum x^2 + eps)^-1/2:  dx = r (dx_hat - x_hat (x_hat . dx_hat))
            def l2norm_bwd(x, xn, dxn):
                r = torch.rsqrt(x.float().pow(2).sum(-1, keepdim=True) + 1e-6)
                xn, dxn = xn.float(), dxn.float()
                return (r * (dxn - xn * (xn * dxn).sum(-1, keepdim=True))).to(x.dtype)
            dq, dk = l2norm_bwd(q, qn, dq), l2norm_bwd(k, kn, dk)
        dA_log = ddt = None
        if use_gate:
            x = g_in.float() + dt_bias.float()
            coef = -torch.exp(A_log.float())
            gval = coef * torch.nn.functional.softplus(x)  # softplus with beta 1, threshold 20 (the kernel's)
            da = dg * coef * torch.where(x <= 20.0, torch.sigmoid(x), torch.ones_like(x))
            dA_log = (dg * gval).sum(dim=(0, 1)).to(A_log.dtype)
            ddt = da.sum(dim=(0, 1)).to(dt_bias.dtype)
            dg = da
        if use_beta_sigmoid:
            db = db * beta * (1.0 - beta)
        if dh0 is not None and initial_state is not None:
            dh0 = dh0.to(initial_state.dtype)
        return (dq, dk, dv, dg.to(g_in.dtype), db.to(beta_in.dtype), dA_log, ddt, None, dh0, None, None, None, None,
                None, None)


@torch.compiler.disable
def chunk_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    cu_seqlens: Optional[torch.Tensor] = None,
    head_first: bool = False,
    transpose_state_layout: bool = False,
    use_gate_in_kernel: bool = False,
    A_log: Optional[torch.Tensor] = None,
    dt_bias: Optional[torch.Tensor] = None,
    use_beta_sigmoid_in_kernel: bool = False,
    output_norm_gate: Optional[torch.Tensor] = None,
    output_norm_weight: Optional[torch.Tensor] = None,
    output_norm_eps: float = 1e-6,
):
    """``(o, final_state | None)`` with gradients for q, k, v, g, beta and initial_state
    (reference: chunk/__init__.py:294-350).  Additions after the reference's surface: with
    ``use_gate_in_kernel`` the argument ``g`` is the raw gate input and
    ``g = -exp(A_log) * softplus(g + dt_bias)`` (``A_log``, ``dt_bias`` ``[Hv]``) is applied here; with
    ``use_beta_sigmoid_in_kernel`` the argument ``beta`` holds logits.  These and ``use_qk_l2norm_in_kernel`` are
    folded into the forward kernels with and without gradients (gradients also reach ``A_log`` and ``dt_bias``).
    With ``output_norm_gate`` ``z`` and ``output_norm_weight`` the returned ``o`` has passed the gated RMS norm
    that follows the op in a GDN layer, ``o * rsqrt(mean(o^2) + eps) * weight * silu(z)``: inside the scan kernel
    when no gradient is needed, as differentiable torch operations behind the op otherwise."""
    assert not head_first, "head_first=True is not supported"
    assert q.dtype == k.dtype == v.dtype
    assert q.dtype != torch.float32, "ChunkGatedDeltaRuleFunction does not support float32. Please use bfloat16."
    if cu_seqlens is not None and q.shape[0] != 1:
        raise ValueError(
            f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
            "Please flatten variable-length inputs before processing.")
    if scale is None:
        scale = k.shape[-1] ** -0.5
    if use_gate_in_kernel and (A_log is None or dt_bias is None):
        raise ValueError("use_gate_in_kernel needs A_log and dt_bias")
    if (output_norm_gate is None) != (output_norm_weight is None):
        raise ValueError("output_norm_gate and output_norm_weight go together")
    fused = use_qk_l2norm_in_kernel or use_gate_in_kernel or use_beta_sigmoid_in_kernel
    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad
        for t in (q, k, v, g, beta, initial_state, A_log, dt_bias, output_norm_gate, output_norm_weight))
    if not needs_grad and (fused or output_norm_gate is not None):
        # inference: normalisation, activations and the output norm are folded into the kernels (no extra passes)
        out = chunk_gated_delta_rule_fwd(q, k, v, g, beta, scale=scale, initial_state=initial_state,
                                         cu_seqlens=cu_seqlens, output_final_state=output_final_state,
                                         transpose_state_layout=transpose_state_layout,
                                         use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel,
                                         A_log=A_log if use_gate_in_kernel else None,
                                         dt_bias=dt_bias if use_gate_in_kernel else None,
                                         beta_is_logit=use_beta_sigmoid_in_kernel,
                                         out_norm_gate=output_norm_gate, out_norm_weight=output_norm_weight,
                                         out_norm_eps=output_norm_eps)
        return out[2].to(q.dtype), out[4]
    if fused:
        o, final_state = ChunkGatedDeltaRuleFusedFunction.apply(
            q, k, v, g, beta, A_log if use_gate_in_kernel else None, dt_bias if use_gate_in_kernel else None, scale,
            initial_state, output_final_state, cu_seqlens, transpose_state_layout, use_qk_l2norm_in_kernel,
            use_gate_in_kernel, use_beta_sigmoid_in_kernel)
    else:
        o, final_state = ChunkGatedDeltaRuleFunction.apply(
            q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, transpose_state_layout,
            torch.is_grad_enabled())
    if output_norm_gate is not None:
        of, z = o.float(), output_norm_gate.float()
        o = (of * torch.rsqrt(of.pow(2).mean(-1, keepdim=True) + output_norm_eps) * output_norm_weight.float()
             * torch.nn.functional.silu(z)).to(o.dtype)
    return o, final_state
