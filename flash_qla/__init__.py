"""Import-path shim: ``import flash_qla`` served by the B200 library ``flashqla_b200``.

Callers of the reference write ``from flash_qla import chunk_gated_delta_rule_fwd`` or
``from flash_qla.utils import l2norm`` (flash_qla/__init__.py:6-38, tests/test_gdr.py:18-21,
benchmark/bench_gated_delta_rule.py:25-30).  With this directory on the path those lines work unchanged and
resolve to the sm_100a implementation.  The five public names are looked up on first use, like the reference
does, so that importing the package stays cheap.
"""
from importlib import import_module

__version__ = "0.1.0+b200"

_HOME = {
    "chunk_gated_delta_rule": "flashqla_b200.chunk",
    "chunk_gated_delta_rule_fwd": "flashqla_b200.chunk",
    "chunk_gated_delta_rule_bwd": "flashqla_b200.chunk",
    "fused_sigmoid_gating_delta_rule_update": "flashqla_b200.recurrent",
    "flashqla_recurrent_gdn_update": "flashqla_b200.recurrent",
}
__all__ = sorted(_HOME)


def __getattr__(name):
    home = _HOME.get(name)
    if home is None:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
    value = getattr(import_module(home), name)
    globals()[name] = value
    return value


def __dir__():
    return sorted(set(globals()) | set(_HOME))
