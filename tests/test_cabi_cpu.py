"""CPU: the C-ABI library builds for sm_100a, loads, and exports every declared symbol."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def built_lib():
    from flashqla_b200 import build
    return build.build()


def test_library_builds_and_loads(built_lib):
    from flashqla_b200 import _cabi
    lib = _cabi.lib()
    assert lib.qla_abi_version() == 2
    assert lib.qla_status_string(0) == b"ok"
    assert lib.qla_status_string(-1) == b"invalid argument"


def test_every_declared_symbol_is_exported(built_lib):
    from flashqla_b200 import _cabi
    header = (ROOT / "include" / "flashqla_b200.h").read_text()
    declared = set(re.findall(r"QLA_API\s+[\w\s\*]+?\b(qla_\w+)\s*\(", header))
    assert declared, "no declarations found"
    assert declared == set(_cabi.EXPORTS), (declared, set(_cabi.EXPORTS))
    handle = ctypes.CDLL(str(built_lib))
    for name in declared:
        assert hasattr(handle, name), name


def test_struct_layouts_match_header(built_lib):
    """Field order of the ctypes mirrors follows the header (names in order)."""
    from flashqla_b200 import _cabi
    header = (ROOT / "include" / "flashqla_b200.h").read_text()
    for cls in (_cabi.QlaRecurrentArgs, _cabi.QlaChunkFwdArgs):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (cls.__name__, cls.__name__), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        names = re.findall(r"(\w+)\s*;", body)
        assert names == [f[0] for f in cls._fields_], cls.__name__


def test_argument_validation_without_gpu(built_lib):
    """Host-side checks of the entry point run before any launch, so they work without a GPU."""
    from flashqla_b200 import _cabi
    lib = _cabi.lib()
    assert lib.qla_recurrent_update(None, None) == -1
    a = _cabi.QlaRecurrentArgs(num_seqs=1, total_tokens=1, tokens_per_seq=1, num_k_heads=3, num_v_heads=4)
    assert lib.qla_recurrent_update(a, None) == -1
    assert b"divisible" in lib.qla_last_error()


def test_python_api_rejects_bad_inputs():
    import flashqla_b200 as fq
    q = torch.zeros(2, 4, 1, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="flattened"):
        fq.fused_sigmoid_gating_delta_rule_update(None, None, None, q, q, q, None, None)
    q = torch.zeros(1, 4, 1, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="CUDA"):
        fq.fused_sigmoid_gating_delta_rule_update(None, None, None, q, q, q, None, None)


def test_manifest_describes_the_header(built_lib):
    """The JSON manifest written beside the library lists every exported function and every argument
    structure with the header's field order, and its offsets are those of the ctypes mirrors."""
    import json
    from flashqla_b200 import _cabi, manifest
    path = built_lib.parent / manifest.MANIFEST_NAME
    assert path.exists(), "the build writes the manifest"
    m = json.loads(path.read_text())
    header = (ROOT / "include" / "flashqla_b200.h").read_text()
    assert m["abi_version"] == int(re.search(r"#define QLA_ABI_VERSION (\d+)", header).group(1))
    assert set(m["exports"]) == set(_cabi.EXPORTS)
    for name, desc in m["structs"].items():
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (name, name), header, re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        assert [f["name"] for f in desc["fields"]] == re.findall(r"(\w+)\s*;", body), name
        cls = getattr(_cabi, name)
        assert desc["size"] == ctypes.sizeof(cls)
        assert all(f["offset"] == getattr(cls, f["name"]).offset for f in desc["fields"])
    for flag, value in m["flags"].items():
        c_name = "QLA_" + flag
        assert re.search(r"%s\s*=\s*%d\b|#define %s\s+%d\b" % (c_name, value, c_name, value), header), c_name


def test_manifest_lists_every_kernel_with_its_cubin(built_lib):
    """The build leaves one cubin per translation unit with kernels; the manifest's kernel entries point at
    them and carry launch constants that agree with the library's own (qla_kernel_launch_info)."""
    import json
    from flashqla_b200 import _cabi, manifest
    m = json.loads((built_lib.parent / manifest.MANIFEST_NAME).read_text())
    kernels = m["kernels"]
    assert kernels, "the build records its kernels"
    names = {k["kernel_name"] for k in kernels}
    assert set(manifest.KERNEL_RULES) <= names
    lib = _cabi.lib()
    for k in kernels:
        assert (built_lib.parent / k["cubin"]).exists(), k["cubin"]
        assert k["registers"] and k["export_name"].startswith("_Z")
        if k["kernel_name"] in manifest.KERNEL_RULES:
            block, smem = ctypes.c_int32(), ctypes.c_size_t()
            assert lib.qla_kernel_launch_info(k["kernel_name"].encode(), ctypes.byref(block), ctypes.byref(smem)) == 0
            assert block.value == 32 * k["num_warps"] and smem.value == k["shared"], k["kernel_name"]
    assert lib.qla_kernel_launch_info(b"no_such_kernel", ctypes.byref(block), ctypes.byref(smem)) == -1
