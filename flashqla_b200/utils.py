"""Host helpers: L2 norm, per-device status word, host copies of cu_seqlens.

Reference counterparts: flash_qla/utils/math.py:7-21 (l2norm), flash_qla/utils/index.py:13-63
(tensor_cache, which keeps its arguments alive in the cache entry; here an entry is keyed on storage +
version, so that in-place edits are seen, and holds a weak reference to the tensor it was made from, so that
an address the allocator hands out again for a new tensor never matches an old entry).
"""
from __future__ import annotations

import weakref
from typing import Optional, Dict, List, Tuple

import torch

_STATUS: Dict[int, torch.Tensor] = {}
_SEQLEN_CACHE: Dict[Tuple, Tuple[weakref.ref, List[int]]] = {}
_SEQLEN_CACHE_MAX = 256
_ORDER_CACHE: Dict[Tuple, Tuple[weakref.ref, Optional[torch.Tensor]]] = {}


def l2norm(x: torch.Tensor, dim: int = -1, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(sum(x^2, -1) + eps)`` computed in fp32, returned in x's dtype (reference:
    flash_qla/utils/math.py:14-21; ``dim`` must be the last one, as there)."""
    assert dim in (-1, x.dim() - 1)
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def unpack(x: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    """Packed ``[1, NT, ...]`` -> zero-padded ``[N, max_len, ...]`` (reference: flash_qla/utils/pack.py:7-20)."""
    assert x.shape[0] == 1 and cu_seqlens.dim() == 1
    cu = cu_seqlens.tolist()
    lens = [b - a for a, b in zip(cu[:-1], cu[1:])]
    y = x.new_zeros((len(lens), max(lens), *x.shape[2:]))
    for i, (a, n) in enumerate(zip(cu[:-1], lens)):
        y[i, :n] = x[0, a:a + n]
    return y


def pack(x: torch.Tensor, cu_seqlens: torch.Tensor) -> torch.Tensor:
    """Padded ``[N, T, ...]`` -> packed ``[1, NT, ...]`` (reference: flash_qla/utils/pack.py:23-35)."""
    assert cu_seqlens.dim() == 1
    cu = cu_seqlens.tolist()
    return torch.cat([x[i, :b - a] for i, (a, b) in enumerate(zip(cu[:-1], cu[1:]))], dim=0).unsqueeze(0)


def pad_and_reshape(x: torch.Tensor, dim: int, chunk_size: int = 64) -> torch.Tensor:
    """Zero-pad ``dim`` to a multiple of ``chunk_size`` and split it into ``[chunks, chunk_size]``
    (reference: flash_qla/utils/pack.py:38-50)."""
    pad = (-x.shape[dim]) % chunk_size
    if pad:
        x = torch.cat([x, x.new_zeros(*x.shape[:dim], pad, *x.shape[dim + 1:])], dim=dim)
    return x.reshape(*x.shape[:dim], -1, chunk_size, *x.shape[dim + 1:])


def fill_last_chunk_of_g(g: torch.Tensor, num_tokens: int, cu_seqlens, chunk_size: int = 64, reverse: bool = False):
    """In place, on chunked gates ``[N, chunks, chunk_size, ...]``: the padded tail of a sequence's last chunk
    repeats the last valid cumulative gate; with ``reverse`` the value accumulated at the last padded position
    is added to the last valid one instead (reference: flash_qla/utils/pack.py:53-83)."""
    if cu_seqlens is None:
        ends = [(slice(None), num_tokens)]
    else:
        cu = cu_seqlens.tolist()
        ends = [(i, b - a) for i, (a, b) in enumerate(zip(cu[:-1], cu[1:]))]
    for row, n in ends:
        c, r = (n // chunk_size, n % chunk_size) if cu_seqlens is not None else (-1, n % chunk_size)
        if r > 0:
            if reverse:
                g[row, c, r - 1] += g[row, c, -1]
            else:
                g[row, c, r:] = g[row, c, r - 1:r]
    return g


def prepare_chunk_offsets(cu_seqlens: torch.Tensor, chunk_size: int) -> torch.Tensor:
    """First chunk index of every sequence, ``[N + 1]`` in cu_seqlens' dtype, computed on cu_seqlens' device
    without a host copy (reference: flash_qla/utils/index.py:122-138)."""
    chunks = (torch.diff(cu_seqlens) + chunk_size - 1) // chunk_size
    return torch.cat([cu_seqlens.new_zeros(1), chunks.cumsum(0)]).to(cu_seqlens.dtype)


def prepare_chunk_indices(cu_seqlens: torch.Tensor, chunk_size: int) -> torch.Tensor:
    """``[total_chunks, 2]`` rows of (sequence, chunk within the sequence) (reference:
    flash_qla/utils/index.py:71-83)."""
    chunks = ((torch.diff(cu_seqlens) + chunk_size - 1) // chunk_size).tolist()
    seq = torch.cat([torch.full((n,), i) for i, n in enumerate(chunks)])
    idx = torch.cat([torch.arange(n) for n in chunks])
    return torch.stack([seq, idx], 1).to(cu_seqlens)


def profile(func, inputs, wait: int = 50, warmup: int = 50, rep: int = 100) -> dict:
    """Device time per kernel (ms, torch.profiler) plus ``"total"`` = mean ms per call between CUDA events
    (reference: flash_qla/utils/profiler.py:8-25)."""
    acts = [torch.profiler.ProfilerActivity.CPU, torch.profiler.ProfilerActivity.CUDA]
    with torch.profiler.profile(activities=acts,
                                schedule=torch.profiler.schedule(wait=wait, warmup=warmup, active=rep)) as prof:
        for _ in range(wait + warmup + rep):
            func(*inputs)
            prof.step()
    result = {x.key: x.device_time * 1e-3 for x in prof.key_averages()}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(rep):
        func(*inputs)
    e1.record()
    torch.cuda.synchronize()
    result["total"] = e0.elapsed_time(e1) / rep
    return result


def device_status(device: torch.device) -> torch.Tensor:
    """The int32 status word the kernels of this device report faults to (0 = fine)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _STATUS.get(idx)
    if st is None:
        st = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _STATUS[idx] = st
    return st


def check_device_status(device=None) -> None:
    """Synchronise and raise if any kernel launched so far reported a fault (e.g. a bounded
    barrier wait that gave up).  The status word is cleared afterwards."""
    from ._cabi import QlaError
    devs = list(_STATUS) if device is None else [torch.device(device).index or 0]
    for idx in devs:
        st = _STATUS.get(idx)
        if st is None:
            continue
        code = int(st.item())
        if code != 0:
            st.zero_()
            names = {1: "a bounded barrier wait timed out", 2: "an index was out of range",
                     3: "tensor memory was not allocated at column 0"}
            # low byte: what happened; the rest says where (barrier index << 8 | parity << 16 | warp << 20)
            raise QlaError(f"device {idx} reported status {code & 0xFF} (detail {code >> 8:#x}): "
                           f"{names.get(code & 0xFF, 'unknown')}")


def _cache_key(cu_seqlens: torch.Tensor) -> Tuple:
    return (cu_seqlens.data_ptr(), cu_seqlens.numel(), str(cu_seqlens.device), cu_seqlens._version)


def _cache_get(cache: Dict, key: Tuple, cu_seqlens: torch.Tensor):
    """Entry of ``cache`` made from this very tensor object, else ``None``.  The key alone is not enough:
    a freed cu_seqlens gives its address back to the allocator, and the next batch's tensor can land on it
    with the same version counter."""
    hit = cache.get(key)
    if hit is not None and hit[0]() is cu_seqlens:
        return hit
    return None


def selftest_bounded_wait(device=None, limit_ms: float = 20.0) -> None:
    """Launch the library's self-test kernel whose only wait can never complete: after ``limit_ms`` the bounded
    wait gives up and records the fault in the device status word, which ``check_device_status`` then raises."""
    from . import _cabi
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = device_status(dev)
    with torch.cuda.device(dev):
        code = _cabi.lib().qla_selftest_bounded_wait(st.data_ptr(), int(limit_ms * 1e6), _cabi.current_stream(dev))
    _cabi.check(code, "qla_selftest_bounded_wait")


def host_seqlens(cu_seqlens: torch.Tensor, total_tokens: Optional[int] = None) -> List[int]:
    """Sequence lengths as Python ints.  One device-to-host copy per distinct cu_seqlens tensor and content
    version; later calls with the same tensor object hit the cache.  ``total_tokens`` (the packed token
    count of the call) is checked against the last boundary when given."""
    key = _cache_key(cu_seqlens)
    hit = _cache_get(_SEQLEN_CACHE, key, cu_seqlens)
    if hit is None:
        cu = cu_seqlens.detach().to("cpu", torch.int64).tolist()
        lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
        if any(n < 0 for n in lens):
            raise ValueError("cu_seqlens must be non-decreasing")
        if cu and cu[0] != 0:
            raise ValueError("cu_seqlens must start at 0")
        if len(_SEQLEN_CACHE) >= _SEQLEN_CACHE_MAX:
            _SEQLEN_CACHE.pop(next(iter(_SEQLEN_CACHE)))
        _SEQLEN_CACHE[key] = (weakref.ref(cu_seqlens), lens)
    else:
        lens = hit[1]
    if total_tokens is not None and sum(lens) != total_tokens:
        raise ValueError(f"cu_seqlens covers {sum(lens)} tokens but the packed inputs hold {total_tokens}")
    return lens


def longest_first_order(cu_seqlens: torch.Tensor, device: torch.device) -> Optional[torch.Tensor]:
    """Int32 permutation on ``device`` that lists the sequences of ``cu_seqlens`` longest first, or ``None``
    when that changes nothing (one sequence, equal lengths).  The chunk scan hands sequences to the GPU in
    this order, so the longest chains start first instead of forming the tail.  Cached like
    ``host_seqlens``; an entry stays for as long as its cu_seqlens tensor is alive (a captured graph keeps
    both), past the cache limit the permutation is simply rebuilt per call."""
    key = _cache_key(cu_seqlens) + (str(device),)
    hit = _cache_get(_ORDER_CACHE, key, cu_seqlens)
    if hit is not None:
        return hit[1]
    lens = host_seqlens(cu_seqlens)
    order = None
    if len(lens) > 1 and min(lens) != max(lens):
        idx = sorted(range(len(lens)), key=lambda i: -lens[i])
        order = torch.tensor(idx, dtype=torch.int32, device=device)
    if len(_ORDER_CACHE) >= _SEQLEN_CACHE_MAX:  # only entries whose cu_seqlens is gone may be dropped
        for dead in [k for k, (ref, _) in _ORDER_CACHE.items() if ref() is None]:
            del _ORDER_CACHE[dead]
    if len(_ORDER_CACHE) < _SEQLEN_CACHE_MAX:
        _ORDER_CACHE[key] = (weakref.ref(cu_seqlens), order)
    return order
