"""Forward for inputs that live in (pinned) host memory.

The reference's entry points take device tensors; a caller whose activations sit on the host pays
host->device copy, compute and device->host copy one after the other.  The recurrence carries nothing but
the fp32 state from one token to the next (``initial_state`` / ``final_state`` of
``chunk_gated_delta_rule_fwd``, flash_qla/ops/gated_delta_rule/chunk/__init__.py:23-86), so one sequence can
be cut into pieces of whole chunks and the three legs overlapped on three CUDA streams: piece p+1 is copied
in while piece p is computed and the output of piece p-1 is copied out.  PCIe is full duplex, so the call
takes about as long as the larger of the two copies instead of their sum.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .chunk import CHUNK, chunk_gated_delta_rule_fwd

_NAMES = ("q", "k", "v", "g", "beta")
_STREAMS = {}


def _copy_streams(dev: torch.device):
    """The two copy streams of a device, created once (stream creation is not free on a per-call path)."""
    key = (dev.type, dev.index)
    if key not in _STREAMS:
        _STREAMS[key] = (torch.cuda.Stream(dev), torch.cuda.Stream(dev))
    return _STREAMS[key]


def chunk_gated_delta_rule_fwd_host(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    final_state_out: Optional[torch.Tensor] = None,
    device: Optional[torch.device] = None,
    piece_tokens: Optional[int] = None,
    transpose_state_layout: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(o, final_state)`` on the host for host tensors ``q, k [1,T,Hk,128]``, ``v [1,T,Hv,128]``,
    ``g, beta [1,T,Hv]``.  ``out`` / ``final_state_out`` are optional preallocated (pinned) host results.
    One sequence per call (``B == 1``); pieces are multiples of the 64-token chunk, so the chunking of the
    sequence - and with it the arithmetic - is that of a single call on the whole sequence.  Pageable
    (non-pinned) inputs work but their copies do not overlap with anything.  ``piece_tokens`` defaults to 8192
    tokens or what 32 MiB of inputs hold, whichever is more: with few heads (a head shard of a multi-GPU run) a
    piece must stay large enough that its copy takes longer than the host needs to issue a piece."""
    if q.is_cuda:
        raise ValueError("chunk_gated_delta_rule_fwd_host takes host tensors; use chunk_gated_delta_rule_fwd")
    if q.shape[0] != 1:
        raise ValueError(f"one sequence per call: the batch size is expected to be 1 rather than {q.shape[0]}")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    T, Hv = q.shape[1], v.shape[2]
    host = dict(q=q, k=k, v=v, g=g, beta=beta)
    in_bytes_per_token = sum(t.numel() * t.element_size() for t in host.values()) // max(T, 1)
    if piece_tokens is None:
        piece_tokens = max(8192, (32 << 20) // max(in_bytes_per_token, 1))
    piece = max(CHUNK, (piece_tokens // CHUNK) * CHUNK)
    tail_tokens = max(1024, (4 << 20) // max(in_bytes_per_token, 1))  # stop halving the tail below ~4 MiB
    if out is None:
        out = torch.empty(v.shape, dtype=v.dtype).pin_memory()
    if final_state_out is None:
        final_state_out = torch.empty(1, Hv, 128, 128, dtype=torch.float32).pin_memory()

    compute = torch.cuda.current_stream(dev)
    copy_in, copy_out = _copy_streams(dev)
    copy_in.wait_stream(compute)
    copy_out.wait_stream(compute)
    state = None if initial_state is None else initial_state.to(dev, torch.float32, non_blocking=True)
    # two sets of device input buffers; a set is refilled once the piece that used it has been computed
    bufs = [{n: torch.empty((1, piece) + tuple(host[n].shape[2:]), dtype=host[n].dtype, device=dev) for n in _NAMES}
            for _ in range(2)]
    computed = [None, None]   # event: the forward that read buffer set s has finished
    keep = []                 # device outputs stay referenced until their copy-out has been waited for
    # Equal pieces, except that the last one is cut in halves down to about a thousand tokens: what cannot
    # overlap with anything is the compute and copy-out of the very last piece, so that one should be small.
    cuts, t0 = [], 0
    while T - t0 > piece:
        cuts.append((t0, piece))
        t0 += piece
    rest = T - t0
    while rest > tail_tokens:
        n = ((rest // 2 + CHUNK - 1) // CHUNK) * CHUNK
        cuts.append((t0, n))
        t0, rest = t0 + n, rest - n
    if rest > 0:
        cuts.append((t0, rest))
    def issue_copy_in(p):
        t0, n = cuts[p]
        s = p & 1
        with torch.cuda.stream(copy_in):
            if computed[s] is not None:
                copy_in.wait_event(computed[s])
            d = {}
            for name in _NAMES:
                d[name] = bufs[s][name][:, :n]
                d[name].copy_(host[name][:, t0:t0 + n], non_blocking=True)
            loaded = torch.cuda.Event()
            loaded.record(copy_in)
        return d, loaded

    # The copy of piece p + 1 is issued BEFORE the forward of piece p: issuing a forward keeps the host busy for
    # longer than a small piece needs on the bus, and the copy engine must not wait for that.
    nxt = issue_copy_in(0)
    for p, (t0, n) in enumerate(cuts):
        s = p & 1
        d, loaded = nxt
        if p + 1 < len(cuts):
            nxt = issue_copy_in(p + 1)
        compute.wait_event(loaded)
        _, _, o, _, state = chunk_gated_delta_rule_fwd(
            d["q"], d["k"], d["v"], d["g"], d["beta"], scale=scale, initial_state=state,
            output_final_state=True, transpose_state_layout=transpose_state_layout)
        computed[s] = torch.cuda.Event()
        computed[s].record(compute)
        keep.append(o)
        with torch.cuda.stream(copy_out):
            copy_out.wait_event(computed[s])
            out[:, t0:t0 + n].copy_(o, non_blocking=True)
    with torch.cuda.stream(copy_out):
        final_state_out.copy_(state, non_blocking=True)
    compute.wait_stream(copy_out)
    compute.wait_stream(copy_in)
    compute.synchronize()
    del keep
    return out, final_state_out
