"""CUDA-graph replay of the chunked forward for callers with static buffers.

One forward call is nine launches of this library plus a few tensor allocations; when the GPU's share of
the work is small (a few heads per GPU after sharding, or short sequences) the host needs longer to issue
them than the GPU to run them.  A serving loop that reuses its buffers can capture the call once and replay
it: the arguments (device pointers, extents, tensor maps) are frozen into the graph, so the inputs must be
updated IN PLACE and the outputs are always the same tensors.
"""
from __future__ import annotations

import torch

from .chunk import chunk_gated_delta_rule_fwd


class GraphedForward:
    """``GraphedForward(q, k, v, g, beta, **kw)`` captures ``chunk_gated_delta_rule_fwd(q, k, v, g, beta, **kw)``;
    calling the object replays it on the current stream and returns the (static) result tuple
    ``(g_cumsum, A, o, h, final_state[, v_new])``.  ``kw`` are the keyword arguments of
    ``chunk_gated_delta_rule_fwd``; tensors among them (``initial_state``, ``cu_seqlens``) are static too."""

    def __init__(self, q, k, v, g, beta, **kw):
        self.inputs = (q, k, v, g, beta)
        self.kw = kw
        # warm-up on a side stream (plans, status words and kernel attributes are set up outside capture)
        side = torch.cuda.Stream(q.device)
        side.wait_stream(torch.cuda.current_stream(q.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                chunk_gated_delta_rule_fwd(q, k, v, g, beta, **kw)
        torch.cuda.current_stream(q.device).wait_stream(side)
        torch.cuda.synchronize(q.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.outputs = chunk_gated_delta_rule_fwd(q, k, v, g, beta, **kw)

    def __call__(self):
        self.graph.replay()
        return self.outputs
