"""Machine-readable description of ``libflashqla_b200.so`` for launchers that are not Python.

The reference's only machine-readable contract is the manifest its AOT export writes next to the sm12x
cubins (``abi_version``, export names, parameter order: flash_qla/compile_sm12x_gdn.py:580-669).  This is the
counterpart for the C ABI of include/flashqla_b200.h: one JSON file beside the shared library with the ABI
version, the target architecture, every exported function with its return and argument types, and every
argument structure with the name, C type, byte offset and size of each field, so that a foreign-function
binding can be generated or checked without parsing the header.  Like the reference's manifest it also has a
``kernels`` list: one entry per compiled kernel with its (mangled) export name, the cubin that holds it
(``cubin/<file>.sm_100a.cubin``, written by the build), warps, dynamic shared memory, registers, the grid rule
and the parameter order, for launchers that load the cubins through the driver API instead of linking the
library.  ``python -m flashqla_b200.manifest`` writes
it; ``flashqla_b200.build`` does so after every link.
"""
from __future__ import annotations

import ctypes as C
import json
import sys
from pathlib import Path

from . import _cabi

MANIFEST_NAME = "libflashqla_b200.manifest.json"

_CTYPE_NAMES = {
    C.c_int: "int", C.c_int32: "int32_t", C.c_int64: "int64_t", C.c_float: "float", C.c_size_t: "size_t",
    C.c_void_p: "void*", C.c_char_p: "const char*", C.c_longlong: "long long",
}

_STRUCTS = (_cabi.QlaRecurrentArgs, _cabi.QlaChunkFwdArgs, _cabi.QlaChunkBwdArgs, _cabi.QlaStateCommitArgs,
            _cabi.QlaCpPlanArgs, _cabi.QlaCpChainArgs)


def _type_name(t) -> str:
    if t is None:
        return "void"
    if t in _CTYPE_NAMES:
        return _CTYPE_NAMES[t]
    if hasattr(t, "_type_") and isinstance(getattr(t, "_type_"), type) and issubclass(t._type_, C.Structure):
        return f"const {t._type_.__name__}*"
    return getattr(t, "__name__", str(t))


# Launch rules of the main kernels: what a launcher has to know besides the cubin.  Block size and dynamic shared
# memory are checked against the library itself (qla_kernel_launch_info) by the tests.
_TMAP = "CUtensorMap (128 B, __grid_constant__)"
KERNEL_RULES = {
    "chunk_fwd_kernel": dict(
        block=384, dynamic_smem=214016, cluster=1, grid="num_seqs * Hv (x 2 with QLA_CHUNK_DUAL_TRANSITION)",
        params=[_TMAP + " q", _TMAP + " k", _TMAP + " v", _TMAP + " A", _TMAP + " w", _TMAP + " o", "FwdParams (by value)"],
        tensor_maps="3-D (width, heads, tokens), 16-bit elements, box 64 x 1 x 64 with 128B swizzle (o: 128 x 1 x 64, none)"),
    "kkt_solve_kernel": dict(
        block=128, dynamic_smem=68608, cluster=1, grid="(pairs of 64-token chunks, Hk)",
        params=[_TMAP + " k", _TMAP + " q", _TMAP + " A", _TMAP + " w", "KktParams (by value)"],
        tensor_maps="3-D (width, heads, tokens), box 64 x 1 x 128 with 128B swizzle"),
    "bwd_scan_kernel": dict(
        block=416, dynamic_smem=214016, cluster=1, grid="num_seqs * Hv (twice that for a dual state-only launch)",
        params=[_TMAP + " q", _TMAP + " k", _TMAP + " dO", _TMAP + " w", _TMAP + " dh (store)", _TMAP + " du (store)",
                "BwdParams (by value)", "BwdScanMode (by value)"],
        tensor_maps="loads: 3-D (width, heads, tokens), box 64 x 1 x 64 with 128B swizzle; stores: workspace rows "
                    "(chunks * Hv * 128) x 128 (dh) or x 64 (du), box 64 x 1 x 128 with 128B swizzle"),
    "bwd_chunk_kernel": dict(
        block=576, dynamic_smem=205824, cluster=1, grid="min(chunks * Hk, SMs), persistent",
        params=[_TMAP + " " + n for n in ("q", "k", "v", "v_new", "dO", "A", "h", "dh", "du", "dq", "dk", "dv")] +
        ["BwdParams (by value)", "int total_items"],
        tensor_maps="q..A, dq..dv: 3-D (width, heads, tokens), box 64 x 1 x 64; h, dh, du: rows of [chunks * Hv * 128, width], box 64 x 1 x 128; all 128B swizzle"),
    "recurrent_kernel": dict(
        block=128, dynamic_smem=32768, cluster=1, grid="min(N * Hv * (128 / rows), resident CTAs), grid-stride over items",
        params=["QlaRecurrentArgs (by value)", "int64 total_items"], tensor_maps=None),
}


def _kernel_entries(directory: Path) -> list:
    """Per-kernel entries from what the build recorded (``kernels.ptxas.json``: the compiler's own report)."""
    rec = Path(directory) / "kernels.ptxas.json"
    if not rec.exists():
        return []
    entries = []
    for src, kernels in json.loads(rec.read_text()).items():
        for k in kernels:
            base = next((n for n in KERNEL_RULES if n in k["mangled"]), None)
            rule = KERNEL_RULES.get(base, {})
            entries.append({
                "export_name": k["mangled"], "kernel_name": base or k["mangled"], "source": src,
                "cubin": f"cubin/{Path(src).stem}.sm_100a.cubin",
                "num_warps": rule["block"] // 32 if rule else None, "num_ctas": rule.get("cluster", 1),
                "shared": rule.get("dynamic_smem"), "static_shared": k["static_smem"], "registers": k["registers"],
                "grid": rule.get("grid"), "param_names": rule.get("params"), "tensor_maps": rule.get("tensor_maps"),
                "launch_cooperative_grid": False, "launch_pdl": False,
            })
    return entries


def describe(directory: Path | None = None) -> dict:
    """The manifest as a dict (no library load: built from the ctypes mirror of the header and the build's
    record of the compiled kernels)."""
    structs = {}
    for s in _STRUCTS:
        structs[s.__name__] = {
            "size": C.sizeof(s),
            "fields": [{"name": n, "type": _type_name(t), "offset": getattr(s, n).offset, "size": getattr(s, n).size}
                       for n, t in s._fields_],
        }
    exports = {name: {"returns": _type_name(res), "args": [_type_name(a) for a in args]}
               for name, (res, args) in _cabi.EXPORTS.items()}
    flags = {n: getattr(_cabi, n) for n in dir(_cabi) if n.startswith(("CHUNK_", "REC_")) and isinstance(getattr(_cabi, n), int)}
    return {
        "abi_version": 2,
        "library": _cabi.lib_path().name,
        "arch": "sm_100a",
        "stream_argument": "cudaStream_t passed as void*",
        "return_convention": "0 on success, negative QLA_ERR_* otherwise; qla_last_error() holds the message",
        "dtype_codes": {"f32": _cabi.QLA_DT_F32, "bf16": _cabi.QLA_DT_BF16, "f16": _cabi.QLA_DT_F16},
        "flags": flags,
        "exports": exports,
        "structs": structs,
        "kernels": _kernel_entries(directory if directory is not None else _cabi.lib_path().parent),
    }


def write_manifest(directory: Path | None = None) -> Path:
    path = (Path(directory) if directory is not None else _cabi.lib_path().parent) / MANIFEST_NAME
    path.parent.mkdir(exist_ok=True)
    path.write_text(json.dumps(describe(path.parent), indent=1) + "\n")
    return path


if __name__ == "__main__":
    print(write_manifest(Path(sys.argv[1]) if len(sys.argv) > 1 else None))
