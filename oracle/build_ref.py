"""Place the reference's own CPU forward / backward beside the oracle, for validation and for the timed CPU arm.

The reference's fp32 PyTorch restatement of the chunked algorithm lives in its test tree (``tests/ref_gdr.py``);
it is plain Python, so "building" it is a copy: from a checkout of the reference into ``oracle/_ref/`` (ignored
by git, never part of the source history).  ``python oracle/build_ref.py [/path/to/FlashQLA]``; without a
checkout nothing happens and the oracle port stands in.  The file imports ``flash_qla.utils`` for its packing
helpers, which the ``flash_qla`` import path of this repository provides.

The reference's recurrent op (``flash_qla/ops/gated_delta_rule/recurrent_fused.py``, TileLang kernels compiled at
run time) is placed there too: ``bench.py --workload decode`` loads it by path as a same-box bar when it is present
and TileLang can compile it for the GPU at hand.  It is never imported by the library.
"""
import shutil
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
DEFAULT_CHECKOUT = Path("/root/reference")


def build(checkout: Path = DEFAULT_CHECKOUT) -> Path | None:
    src = Path(checkout) / "tests" / "ref_gdr.py"
    if not src.exists():
        return None
    dst = HERE / "_ref" / "ref_gdr.py"
    dst.parent.mkdir(exist_ok=True)
    shutil.copyfile(src, dst)
    rec = Path(checkout) / "flash_qla" / "ops" / "gated_delta_rule" / "recurrent_fused.py"
    if rec.exists():
        shutil.copyfile(rec, HERE / "_ref" / "recurrent_fused.py")
    return dst


if __name__ == "__main__":
    print(build(Path(sys.argv[1]) if len(sys.argv) > 1 else DEFAULT_CHECKOUT))
