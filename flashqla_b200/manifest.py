"""Machine-readable description of ``libflashqla_b200.so`` for launchers that are not Python.

The reference's only machine-readable contract is the manifest its AOT export writes next to the sm12x
cubins (``abi_version``, export names, parameter order: flash_qla/compile_sm12x_gdn.py:580-669).  This is the
counterpart for the C ABI of include/flashqla_b200.h: one JSON file beside the shared library with the ABI
version, the target architecture, every exported function with its return and argument types, and every
argument structure with the name, C type, byte offset and size of each field, so that a foreign-function
binding can be generated or checked without parsing the header.  ``python -m flashqla_b200.manifest`` writes
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


def describe() -> dict:
    """The manifest as a dict (no library load: built from the ctypes mirror of the header)."""
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
    }


def write_manifest(directory: Path | None = None) -> Path:
    path = (Path(directory) if directory is not None else _cabi.lib_path().parent) / MANIFEST_NAME
    path.parent.mkdir(exist_ok=True)
    path.write_text(json.dumps(describe(), indent=1) + "\n")
    return path


if __name__ == "__main__":
    print(write_manifest(Path(sys.argv[1]) if len(sys.argv) > 1 else None))
