"""Gate-driven intra-card context parallelism (CP) for the chunked forward.

Host-side mirror of flash_qla/ops/gated_delta_rule/chunk/cp_context.py: ``_calc_cp_seqs`` (:36-114,
the planner) and ``intra_card_cp_preprocess`` (:117-176, the warm-up / chaining sequence).  The
planner's constants are re-derived for B200 (148 SMs, one resident chunk-scan CTA per SM):

* CP is used when the (sequence, v-head) chains alone cannot fill the machine:
  ``chains < 2 * SMs`` and some sequence is long enough to be cut.
* The segment length minimises an estimate of the makespan.  One scan CTA is resident per SM and CTAs
  are handed to SMs as they free up, so the main scan takes ``ceil(CTAs / SMs)`` rounds of one segment
  each; the warm-up pass costs another ``WARMUP_CHUNKS`` state-only chunks per round.  What matters
  is therefore how close ``CTAs / SMs`` comes to an integer from below, not how small the segments are
  (19 segments x 32 heads = 4.1 rounds is far worse than 9 x 32 = 1.95 rounds).  Floor of
  ``MIN_SEG_CHUNKS`` chunks per segment.

Everything that depends on tensor VALUES (warm-up lengths, fallback heads) is decided on the device
(``qla_cp_plan``); the host plan depends on the sequence LENGTHS only, so a cached plan never needs a
device-to-host copy.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import _cabi

CHUNK = 64
MIN_SEG_CHUNKS = 8
WARMUP_CHUNKS = 10        # typical length of the warm-up pass (chunks until the decay passes the threshold)
WARMUP_COST = 0.6         # cost of a state-only chunk relative to a full one
WARMUP_THRESHOLD = -10.0
INLINE_WARMUP = True      # fold the warm-up of a segment into its own scan where no transition matrix is needed  # exp(-10) ~ 4.5e-5: what a dropped prefix may contribute (cp_fwd.py:29-61)


@dataclass
class CpPlan:
    use_cp: bool
    seg_chunks: int = 0
    cu: Optional[List[int]] = None           # segment boundaries, len = n_seg + 1
    seg_next: Optional[List[int]] = None     # successor segment or -1
    seg_raw: Optional[List[int]] = None      # raw sequence of a segment that ENDS it, else -1
    raw_first: Optional[List[int]] = None    # first segment of every raw sequence, len = n_raw + 1
    dev: Optional[Dict[str, torch.Tensor]] = None
    tables: Optional[Dict[str, torch.Tensor]] = None  # chunk-table workspace of `cu`, built with the plan


_PLAN_CACHE: Dict[Tuple, CpPlan] = {}


def plan_segments(lens: Sequence[int], num_v_heads: int, num_sms: int = 148) -> CpPlan:
    """Decide whether to cut sequences and where.  Pure function of lengths, head count, SM count."""
    chunks = [(n + CHUNK - 1) // CHUNK for n in lens]
    chains = len(lens) * num_v_heads
    if not chunks or chains >= 2 * num_sms or max(chunks) < 2 * MIN_SEG_CHUNKS:
        return CpPlan(use_cp=False)
    best, seg = None, 0
    for cand in range(MIN_SEG_CHUNKS, max(chunks)):
        ctas = sum(-(-c // cand) for c in chunks) * num_v_heads
        rounds = -(-ctas // num_sms)
        # the last segment of a sequence may be shorter; the longest one sets the round time
        longest = max(min(c, cand) for c in chunks)
        cost = rounds * (longest + WARMUP_COST * min(WARMUP_CHUNKS, longest))
        if best is None or cost < best:
            best, seg = cost, cand
    uncut = -(-chains // num_sms) * max(chunks)
    if best is None or best >= uncut:
        return CpPlan(use_cp=False)
    cu, seg_next, seg_raw, raw_first = [0], [], [], [0]
    start = 0
    for r, n in enumerate(lens):
        pieces = max(1, -(-chunks[r] // seg))
        for p in range(pieces):
            end_tok = min(n, (p + 1) * seg * CHUNK) if p + 1 < pieces else n
            cu.append(start + end_tok)
            last = p + 1 == pieces
            seg_next.append(-1 if last else len(seg_next) + 1)
            seg_raw.append(r if last else -1)
        start += n
        raw_first.append(len(seg_next))
    return CpPlan(True, seg, cu, seg_next, seg_raw, raw_first)


def get_plan(lens: Sequence[int], num_v_heads: int, device: torch.device) -> CpPlan:
    key = (tuple(lens), num_v_heads, str(device))
    plan = _PLAN_CACHE.get(key)
    if plan is None:
        sms = torch.cuda.get_device_properties(device).multi_processor_count
        plan = plan_segments(lens, num_v_heads, sms)
        if plan.use_cp:
            from .chunk import chunk_tables_workspace
            plan.tables = chunk_tables_workspace(plan.cu, device)
            i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
            n_seg = len(plan.seg_next)
            plan.dev = dict(
                cu=i32(plan.cu), seg_next=i32(plan.seg_next), seg_raw=i32(plan.seg_raw),
                raw_first=i32(plan.raw_first),
                # row of cp_h0 a segment's end state is written to by the warm-up pass
                warm_map=i32([s if s >= 0 else -1 for s in plan.seg_next]),
                identity=i32(list(range(n_seg))),
                # original sequence a segment starts (-1: it continues one)
                seg_start_of=i32([plan.raw_first.index(s) if s in plan.raw_first[:-1] else -1 for s in range(n_seg)]),
                # predecessor segment (-1: the segment starts a sequence): the backward's "next"
                seg_prev=i32([-1 if s in plan.raw_first[:-1] else s - 1 for s in range(n_seg)]))
        # Plans are never evicted: captured CUDA graphs and in-flight launches keep using a plan's device
        # tensors.  Past 256 distinct shapes new plans are simply not cached.
        if len(_PLAN_CACHE) < 256:
            _PLAN_CACHE[key] = plan
    return plan


def segment_initial_states(plan: CpPlan, k, v, beta, g_cumsum, A, w, h0, scale, launch_fwd, rnorm=None,
                           h0_map=None, h0_transposed=False, inline_warmup=None):
    """Run plan (+ start states) -> warm-up and transition passes (one launch) -> chaining.  Returns ``(cp_h0,
    lead)``: ``cp_h0`` fp32 ``[n_seg, Hv, 128(K), 128(V)]`` is the state a segment starts from, ``lead`` int32
    ``[n_seg, Hv]`` (or ``None``) the number of chunks in front of a segment that the main scan runs first from a
    zero state INSTEAD of reading ``cp_h0`` (the warm-up folded into the scan: every sequence and head whose
    segments all decay below the threshold; the state-only launch then finds nothing to do for them).
    ``launch_fwd`` is ``chunk._launch_fwd``; ``w`` is the prepared chunk operand that goes with ``A``; ``h0`` are
    the caller's initial states (fp32 or bf16, ``[V, K]`` with ``h0_transposed``, rows picked by ``h0_map``)."""
    dev = k.device
    Hv = beta.shape[2]
    d = plan.dev
    n_seg = len(plan.seg_next)
    lib = _cabi.lib()
    stream = _cabi.current_stream(dev)
    warm_limit = torch.empty(n_seg, Hv, dtype=torch.int32, device=dev)
    m_limit = torch.empty(n_seg, Hv, dtype=torch.int32, device=dev)
    cp_h0 = torch.empty(n_seg, Hv, 128, 128, dtype=torch.float32, device=dev)
    if inline_warmup is None:
        inline_warmup = INLINE_WARMUP
    lead = torch.empty(n_seg, Hv, dtype=torch.int32, device=dev) if inline_warmup else None
    pa = _cabi.QlaCpPlanArgs(num_segments=n_seg, num_v_heads=Hv, threshold=WARMUP_THRESHOLD,
                             g_cumsum=g_cumsum.data_ptr(), cu_seqlens=d["cu"].data_ptr(),
                             seg_next=d["seg_next"].data_ptr(), warm_limit=warm_limit.data_ptr(),
                             m_limit=m_limit.data_ptr(), cp_h0=cp_h0.data_ptr(), seg_start_of=d["seg_start_of"].data_ptr(),
                             h0=_cabi.ptr(h0), h0_map=_cabi.ptr(h0_map),
                             h0_dtype=_cabi.dtype_code(h0.dtype) if h0 is not None else 0,
                             h0_transposed=1 if h0_transposed else 0, lead=_cabi.ptr(lead),
                             raw_first_seg=d["raw_first"].data_ptr(), num_raw_seqs=len(plan.raw_first) - 1)
    with torch.cuda.device(dev):
        _cabi.check(lib.qla_cp_plan(pa, stream), "qla_cp_plan")
    # One launch, two passes: segment-end states from the trailing `warm_limit` chunks, written straight into the
    # successor's row, and the transition matrices of the (segment, head) pairs that never decayed below the
    # threshold.
    M = torch.empty(n_seg, Hv, 128, 128, dtype=torch.float32, device=dev)
    launch_fwd(None, k, v, None, beta, None, d["cu"], g_cumsum, A, None, None, None, cp_h0, scale,
               flags=_cabi.CHUNK_STATE_ONLY | _cabi.CHUNK_SKIP_PREPARE, seq_map=d["warm_map"], chunk_limit=warm_limit,
               num_seqs=n_seg, w=w, tables=plan.tables, rnorm=rnorm, dual=(m_limit, d["identity"], M))
    ca = _cabi.QlaCpChainArgs(num_raw_seqs=len(plan.raw_first) - 1, num_v_heads=Hv, h0=cp_h0.data_ptr(),
                              M=M.data_ptr(), m_limit=m_limit.data_ptr(), raw_first_seg=d["raw_first"].data_ptr())
    with torch.cuda.device(dev):
        _cabi.check(lib.qla_cp_chain(ca, stream), "qla_cp_chain")
    return cp_h0, lead


def segment_end_gradients(plan: CpPlan, q, k, do, w, g_cumsum, dht, scale, transposed=False):
    """The backward's counterpart of :func:`segment_initial_states` (the reference's backward has no context
    parallelism: its grid is sequences x heads, chunk/hopper/fused_bwd.py:79).  Returns ``(seg_dht, lead)``:
    ``seg_dht`` fp32 ``[n_seg, Hv, 128(K), 128(V)]`` is the state gradient entering a segment from its right end,
    ``lead`` (or ``None``) the number of chunks behind a segment that its reverse scan runs first from a zero
    gradient instead (the warm-up folded into the scan, as in the forward).

    plan (reverse: decay accumulated from a segment's START; rows of the last segments take the caller's ``dht``)
    -> one launch of the reverse scan in state-only mode over the leading chunks of every segment (zero start,
    result written to the predecessor's row) together with the transition matrices of the pairs whose decay never
    passed the threshold -> reverse chaining."""
    dev = k.device
    Hv = w.shape[2]
    Hk = k.shape[2]
    d = plan.dev
    n_seg = len(plan.seg_next)
    lib = _cabi.lib()
    stream = _cabi.current_stream(dev)
    warm_limit = torch.empty(n_seg, Hv, dtype=torch.int32, device=dev)
    m_limit = torch.empty(n_seg, Hv, dtype=torch.int32, device=dev)
    seg_dht = torch.empty(n_seg, Hv, 128, 128, dtype=torch.float32, device=dev)
    lead = torch.empty(n_seg, Hv, dtype=torch.int32, device=dev) if INLINE_WARMUP else None
    pa = _cabi.QlaCpPlanArgs(num_segments=n_seg, num_v_heads=Hv, threshold=WARMUP_THRESHOLD,
                             g_cumsum=g_cumsum.data_ptr(), cu_seqlens=d["cu"].data_ptr(),
                             seg_next=d["seg_prev"].data_ptr(), warm_limit=warm_limit.data_ptr(),
                             m_limit=m_limit.data_ptr(), cp_h0=seg_dht.data_ptr(), seg_start_of=d["seg_raw"].data_ptr(),
                             h0=_cabi.ptr(dht), h0_map=None, h0_dtype=_cabi.QLA_DT_F32,
                             h0_transposed=1 if transposed else 0, reverse=1, lead=_cabi.ptr(lead),
                             raw_first_seg=d["raw_first"].data_ptr(), num_raw_seqs=len(plan.raw_first) - 1)
    M = torch.empty(n_seg, Hv, 128, 128, dtype=torch.float32, device=dev)
    total = q.shape[0] * q.shape[1]
    from .utils import device_status
    sa = _cabi.QlaChunkBwdArgs(
        batch=1, seq_len=total, num_seqs=n_seg, num_k_heads=Hk, num_v_heads=Hv, qkv_dtype=_cabi.dtype_code(q.dtype),
        beta_dtype=_cabi.QLA_DT_F32, flags=_cabi.CHUNK_STATE_ONLY | _cabi.CHUNK_DUAL_TRANSITION, scale=float(scale),
        q=_cabi.ptr(q), k=_cabi.ptr(k), g_cumsum=_cabi.ptr(g_cumsum), w=_cabi.ptr(w), d_o=_cabi.ptr(do),
        cu_seqlens=d["cu"].data_ptr(), dh0=seg_dht.data_ptr(), status=_cabi.ptr(device_status(dev)),
        chunk_limit=warm_limit.data_ptr(), out_map=d["seg_prev"].data_ptr(), chunk_limit_b=m_limit.data_ptr(),
        out_map_b=d["identity"].data_ptr(), out_b=M.data_ptr())
    ca = _cabi.QlaCpChainArgs(num_raw_seqs=len(plan.raw_first) - 1, num_v_heads=Hv, h0=seg_dht.data_ptr(),
                              M=M.data_ptr(), m_limit=m_limit.data_ptr(), raw_first_seg=d["raw_first"].data_ptr(),
                              reverse=1)
    with torch.cuda.device(dev):
        _cabi.check(lib.qla_cp_plan(pa, stream), "qla_cp_plan")
        _cabi.check(lib.qla_chunk_bwd(sa, stream), "qla_chunk_bwd (state-only)")
        _cabi.check(lib.qla_cp_chain(ca, stream), "qla_cp_chain")
    return seg_dht, lead
