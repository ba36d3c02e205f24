"""Build ``libflashqla_b200.so`` (the C-ABI library of include/flashqla_b200.h) with nvcc for sm_100a.

The library is built in-tree (``flashqla_b200/_lib/``) so that it travels with the source tree;
nothing is JIT-compiled at run time.  ``python -m flashqla_b200.build`` rebuilds it.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "_lib"
LIB_PATH = LIB_DIR / "libflashqla_b200.so"
STAMP = LIB_DIR / "build.stamp"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    "-DQLA_BUILDING_LIB",
]


def _extra_flags() -> list[str]:
    """Extra nvcc flags for experiments (``QLA_NVCC_EXTRA="-DQLA_REC_REG_PREFETCH=0"``); empty in normal builds."""
    return os.environ.get("QLA_NVCC_EXTRA", "").split()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _digest() -> str:
    h = hashlib.sha256()
    for f in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) +
                    [PKG.parent / "include" / "flashqla_b200.h", Path(__file__)]):
        h.update(f.name.encode())
        h.update(f.read_bytes())
    return h.hexdigest()


def is_current() -> bool:
    return LIB_PATH.exists() and STAMP.exists() and STAMP.read_text().strip() == _digest()


KERNELS_JSON = LIB_DIR / "kernels.ptxas.json"
CUBIN_DIR = LIB_DIR / "cubin"


def _parse_ptxas(log: str) -> list[dict]:
    """Entry functions of one translation unit from the ``-Xptxas -v`` log: mangled name, registers, static
    shared memory, spills (what the compiler itself reports; no binary is inspected)."""
    import re
    out, cur = [], None
    for line in log.splitlines():
        m = re.search(r"Compiling entry function '([^']+)' for 'sm_100a'", line)
        if m:
            cur = {"mangled": m.group(1), "registers": None, "static_smem": 0, "spill_stores": 0}
            out.append(cur)
            continue
        if cur is None:
            continue
        m = re.search(r"(\d+) bytes spill stores", line)
        if m:
            cur["spill_stores"] = int(m.group(1))
        m = re.search(r"Used (\d+) registers", line)
        if m:
            cur["registers"] = int(m.group(1))
            sm = re.search(r"(\d+) bytes smem", line)
            cur["static_smem"] = int(sm.group(1)) if sm else 0
            cur = None
    return out


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` and link the shared library; beside it one cubin per translation unit with
    kernels (for launchers that load kernels without the CUDA runtime) and the manifest.  Returns the library's
    path."""
    import json
    if not force and is_current():
        from .manifest import MANIFEST_NAME, write_manifest
        if not (LIB_DIR / MANIFEST_NAME).exists():
            write_manifest(LIB_DIR)
        return LIB_PATH
    LIB_DIR.mkdir(exist_ok=True)
    CUBIN_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    objs = []
    procs = []
    for src in sources():
        obj = LIB_DIR / (src.stem + ".o")
        cmd = [nvcc, "-Xptxas", "-v", *NVCC_FLAGS, *_extra_flags(), "-c", str(src), "-o", str(obj)]
        procs.append((src, "obj", subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
        cubin = CUBIN_DIR / (src.stem + ".sm_100a.cubin")
        cmd = [nvcc, *[f for f in NVCC_FLAGS if f not in ("-Xcompiler", "-fPIC", "-fvisibility=hidden")], "-cubin",
               str(src), "-o", str(cubin)]
        procs.append((src, "cubin", subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed, kernels = [], {}
    for src, kind, pr in procs:
        out, _ = pr.communicate()
        if verbose or pr.returncode != 0:
            sys.stderr.write(f"--- {src.name} ({kind})\n{out}\n")
        if pr.returncode != 0:
            failed.append(f"{src.name} ({kind})")
        elif kind == "obj":
            entries = _parse_ptxas(out)
            if entries:
                kernels[src.name] = entries
    if failed:
        raise RuntimeError(f"nvcc failed for: {', '.join(failed)}")
    for src in sources():  # translation units without kernels leave no cubin behind
        if src.name not in kernels:
            (CUBIN_DIR / (src.stem + ".sm_100a.cubin")).unlink(missing_ok=True)
    link = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-gencode",
            "arch=compute_100a,code=sm_100a", "-lcudart"]
    subprocess.run(link, check=True)
    KERNELS_JSON.write_text(json.dumps(kernels, indent=1) + "\n")
    STAMP.write_text(_digest())
    from .manifest import write_manifest  # JSON description of the exports and kernels beside the library
    write_manifest(LIB_DIR)
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
