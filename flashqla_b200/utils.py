"""Host helpers: L2 norm, per-device status word, host copies of cu_seqlens.

Reference counterparts: flash_qla/utils/math.py:7-21 (l2norm), flash_qla/utils/index.py:13-63
(tensor_cache, keyed on object identity there; keyed on storage + version here so that in-place edits
are seen).
"""
from __future__ import annotations

from typing import Optional, Dict, List, Tuple

import torch

_STATUS: Dict[int, torch.Tensor] = {}
_SEQLEN_CACHE: Dict[Tuple, List[int]] = {}
_SEQLEN_CACHE_MAX = 256
_ORDER_CACHE: Dict[Tuple, Optional[torch.Tensor]] = {}


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """``x * rsqrt(sum(x^2, -1) + eps)`` computed in fp32, returned in x's dtype."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


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


def host_seqlens(cu_seqlens: torch.Tensor) -> List[int]:
    """Sequence lengths as Python ints.  One device-to-host copy per distinct cu_seqlens content
    version; later calls with the same tensor hit the cache."""
    key = (cu_seqlens.data_ptr(), cu_seqlens.numel(), str(cu_seqlens.device), cu_seqlens._version)
    lens = _SEQLEN_CACHE.get(key)
    if lens is None:
        cu = cu_seqlens.detach().to("cpu", torch.int64).tolist()
        lens = [cu[i + 1] - cu[i] for i in range(len(cu) - 1)]
        if any(n < 0 for n in lens):
            raise ValueError("cu_seqlens must be non-decreasing")
        if len(_SEQLEN_CACHE) >= _SEQLEN_CACHE_MAX:
            _SEQLEN_CACHE.pop(next(iter(_SEQLEN_CACHE)))
        _SEQLEN_CACHE[key] = lens
    return lens


def longest_first_order(cu_seqlens: torch.Tensor, device: torch.device) -> Optional[torch.Tensor]:
    """Int32 permutation on ``device`` that lists the sequences of ``cu_seqlens`` longest first, or ``None``
    when that changes nothing (one sequence, equal lengths).  The chunk scan hands sequences to the GPU in
    this order, so the longest chains start first instead of forming the tail.  Cached like
    ``host_seqlens``; entries are never evicted (launches in flight and captured graphs use the tensor), past
    the cache limit the permutation is simply rebuilt per call."""
    key = (cu_seqlens.data_ptr(), cu_seqlens.numel(), str(cu_seqlens.device), cu_seqlens._version, str(device))
    if key in _ORDER_CACHE:
        return _ORDER_CACHE[key]
    lens = host_seqlens(cu_seqlens)
    order = None
    if len(lens) > 1 and min(lens) != max(lens):
        idx = sorted(range(len(lens)), key=lambda i: -lens[i])
        order = torch.tensor(idx, dtype=torch.int32, device=device)
    if len(_ORDER_CACHE) < _SEQLEN_CACHE_MAX:
        _ORDER_CACHE[key] = order
    return order
