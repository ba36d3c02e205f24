"""ctypes binding of ``libflashqla_b200.so`` (include/flashqla_b200.h).

The library is the product: there is no Python / CPU fallback.  ``lib()`` raises if the shared
object has not been built (``python -m flashqla_b200.build``).
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libflashqla_b200.so"
_lib = None

QLA_DT_F32, QLA_DT_BF16, QLA_DT_F16 = 0, 1, 2
_DTYPES = {torch.float32: QLA_DT_F32, torch.bfloat16: QLA_DT_BF16, torch.float16: QLA_DT_F16}

REC_QK_L2NORM, REC_DISABLE_STATE_UPDATE, REC_A_IS_LOG_DECAY, REC_B_IS_BETA = 1, 2, 4, 8
CHUNK_TRANSPOSE_STATE, CHUNK_STATE_ONLY, CHUNK_QK_L2NORM, CHUNK_SKIP_PREPARE = 1, 2, 4, 8
CHUNK_INIT_IDENTITY, CHUNK_ZERO_V, CHUNK_PREPARE_ONLY, CHUNK_A_GIVEN, CHUNK_TABLES_READY = 16, 32, 64, 128, 256
CHUNK_GATE_ACT, CHUNK_BETA_LOGIT, CHUNK_H0_KV_F32, CHUNK_DUAL_TRANSITION, CHUNK_OUT_GATED_RMSNORM = 512, 1024, 2048, 4096, 8192


class QlaError(RuntimeError):
    """A C-ABI entry point returned a negative status."""


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ValueError(f"unsupported dtype {dt}") from None


class QlaRecurrentArgs(C.Structure):
    _fields_ = [
        ("num_seqs", C.c_int32), ("total_tokens", C.c_int32), ("tokens_per_seq", C.c_int32),
        ("num_k_heads", C.c_int32), ("num_v_heads", C.c_int32), ("qkv_dtype", C.c_int32),
        ("a_dtype", C.c_int32), ("a_log_dtype", C.c_int32), ("dt_bias_dtype", C.c_int32),
        ("inter_dtype", C.c_int32), ("inter_steps", C.c_int32), ("parents_stride", C.c_int32),
        ("flags", C.c_int32), ("rows_per_cta", C.c_int32),
        ("state_slots", C.c_int64), ("inter_slots", C.c_int64),
        ("scale", C.c_float), ("softplus_beta", C.c_float), ("softplus_threshold", C.c_float),
        ("A_log", C.c_void_p), ("a", C.c_void_p), ("dt_bias", C.c_void_p), ("q", C.c_void_p),
        ("k", C.c_void_p), ("v", C.c_void_p), ("b", C.c_void_p), ("state", C.c_void_p),
        ("state_indices", C.c_void_p), ("cu_seqlens", C.c_void_p), ("inter", C.c_void_p),
        ("inter_indices", C.c_void_p), ("parents", C.c_void_p), ("o", C.c_void_p),
        ("status", C.c_void_p), ("state_dtype", C.c_int32), ("parents_steps", C.c_int32),
    ]


class QlaChunkFwdArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seq_len", C.c_int32), ("num_seqs", C.c_int32),
        ("num_k_heads", C.c_int32), ("num_v_heads", C.c_int32), ("qkv_dtype", C.c_int32),
        ("gate_dtype", C.c_int32), ("beta_dtype", C.c_int32), ("flags", C.c_int32),
        ("max_chunks_per_seq", C.c_int32), ("scale", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p),
        ("beta", C.c_void_p), ("h0", C.c_void_p), ("cu_seqlens", C.c_void_p),
        ("seq_map", C.c_void_p), ("seq_order", C.c_void_p), ("chunk_limit", C.c_void_p), ("g_cumsum", C.c_void_p), ("A", C.c_void_p), ("w", C.c_void_p),
        ("qk_rnorm", C.c_void_p), ("A_log", C.c_void_p), ("dt_bias", C.c_void_p), ("beta_out", C.c_void_p), ("o", C.c_void_p), ("h", C.c_void_p), ("v_new", C.c_void_p), ("final_state", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
        ("h0_map", C.c_void_p), ("state_dtype", C.c_int32), ("reserved", C.c_int32),
        ("chunk_limit_b", C.c_void_p), ("seq_map_b", C.c_void_p), ("final_state_b", C.c_void_p),
        ("norm_gate", C.c_void_p), ("norm_weight", C.c_void_p), ("norm_eps", C.c_float), ("reserved2", C.c_int32),
        ("lead", C.c_void_p),
    ]


class QlaChunkBwdArgs(C.Structure):
    _fields_ = [
        ("batch", C.c_int32), ("seq_len", C.c_int32), ("num_seqs", C.c_int32),
        ("num_k_heads", C.c_int32), ("num_v_heads", C.c_int32), ("qkv_dtype", C.c_int32),
        ("beta_dtype", C.c_int32), ("flags", C.c_int32), ("scale", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g_cumsum", C.c_void_p),
        ("beta", C.c_void_p), ("A", C.c_void_p), ("h", C.c_void_p), ("v_new", C.c_void_p),
        ("w", C.c_void_p), ("d_o", C.c_void_p), ("dht", C.c_void_p), ("cu_seqlens", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("dbeta", C.c_void_p),
        ("dg", C.c_void_p), ("dh0", C.c_void_p), ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
        ("num_segments", C.c_int32), ("reserved", C.c_int32), ("seg_cu", C.c_void_p), ("seg_dht", C.c_void_p),
        ("seg_dh0_map", C.c_void_p), ("chunk_limit", C.c_void_p), ("out_map", C.c_void_p),
        ("chunk_limit_b", C.c_void_p), ("out_map_b", C.c_void_p), ("out_b", C.c_void_p), ("seg_lead", C.c_void_p),
    ]


class QlaStateCommitArgs(C.Structure):
    _fields_ = [
        ("num_seqs", C.c_int32), ("num_v_heads", C.c_int32), ("inter_dtype", C.c_int32), ("inter_steps", C.c_int32),
        ("inter_slots", C.c_int64), ("state_slots", C.c_int64), ("inter", C.c_void_p), ("accepted", C.c_void_p),
        ("state_indices", C.c_void_p), ("inter_indices", C.c_void_p), ("state", C.c_void_p), ("status", C.c_void_p),
        ("state_dtype", C.c_int32), ("reserved", C.c_int32),
    ]


class QlaCpPlanArgs(C.Structure):
    _fields_ = [
        ("num_segments", C.c_int32), ("num_v_heads", C.c_int32), ("threshold", C.c_float),
        ("g_cumsum", C.c_void_p), ("cu_seqlens", C.c_void_p), ("seg_next", C.c_void_p),
        ("warm_limit", C.c_void_p), ("m_limit", C.c_void_p),
        ("cp_h0", C.c_void_p), ("seg_start_of", C.c_void_p), ("h0", C.c_void_p), ("h0_map", C.c_void_p),
        ("h0_dtype", C.c_int32), ("h0_transposed", C.c_int32), ("reverse", C.c_int32), ("num_raw_seqs", C.c_int32),
        ("lead", C.c_void_p), ("raw_first_seg", C.c_void_p),
    ]


class QlaCpChainArgs(C.Structure):
    _fields_ = [
        ("num_raw_seqs", C.c_int32), ("num_v_heads", C.c_int32), ("h0", C.c_void_p), ("M", C.c_void_p),
        ("m_limit", C.c_void_p), ("raw_first_seg", C.c_void_p), ("reverse", C.c_int32), ("reserved", C.c_int32),
    ]


# Every symbol include/flashqla_b200.h declares; tests check that the built library exports each.
EXPORTS = {
    "qla_recurrent_update": (C.c_int, [C.POINTER(QlaRecurrentArgs), C.c_void_p]),
    "qla_state_commit": (C.c_int, [C.POINTER(QlaStateCommitArgs), C.c_void_p]),
    "qla_chunk_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(QlaChunkFwdArgs)]),
    "qla_chunk_fwd": (C.c_int, [C.POINTER(QlaChunkFwdArgs), C.c_void_p]),
    "qla_chunk_fwd_noalloc": (C.c_int, [C.POINTER(QlaChunkFwdArgs), C.c_void_p]),
    "qla_chunk_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(QlaChunkBwdArgs)]),
    "qla_chunk_bwd": (C.c_int, [C.POINTER(QlaChunkBwdArgs), C.c_void_p]),
    "qla_cp_plan": (C.c_int, [C.POINTER(QlaCpPlanArgs), C.c_void_p]),
    "qla_cp_chain": (C.c_int, [C.POINTER(QlaCpChainArgs), C.c_void_p]),
    "qla_set_trace_buffer": (C.c_int, [C.c_void_p, C.c_size_t]),
    "qla_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "qla_kernel_launch_info": (C.c_int, [C.c_char_p, C.POINTER(C.c_int32), C.POINTER(C.c_size_t)]),
    "qla_status_string": (C.c_char_p, [C.c_int]),
    "qla_last_error": (C.c_char_p, []),
    "qla_abi_version": (C.c_int, []),
}


def lib_path() -> Path:
    return _LIB_PATH


def lib():
    """Load the shared library once.  Raises ``QlaError`` when it is missing: the CUDA path is the
    only path."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise QlaError(
                f"{_LIB_PATH} is missing: build it with `python -m flashqla_b200.build` "
                "(nvcc, sm_100a). flashqla_b200 has no CPU or PyTorch fallback.")
        handle = C.CDLL(str(_LIB_PATH))
        for name, (res, argtypes) in EXPORTS.items():
            fn = getattr(handle, name, None)
            if fn is None:
                raise QlaError(f"{_LIB_PATH} does not export {name}; rebuild the library")
            fn.restype, fn.argtypes = res, argtypes
        _lib = handle
    return _lib


def check(code: int, what: str) -> None:
    if code != 0:
        handle = lib()
        detail = handle.qla_last_error().decode(errors="replace")
        status = handle.qla_status_string(code).decode()
        if code in (-1,):
            raise ValueError(f"{what}: {status}: {detail}")
        if code == -2:
            raise NotImplementedError(f"{what}: {status}: {detail}")
        raise QlaError(f"{what}: {status}: {detail}")


def ptr(t) -> int | None:
    return None if t is None else t.data_ptr()


def current_stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
