"""Architecture predicates the reference's callers import (flash_qla/ops/gated_delta_rule/chunk/arch.py:7-20).
This build targets sm_100a only; the predicates answer for the current CUDA device."""
import torch


def get_compute_version() -> str:
    major, minor = torch.cuda.get_device_capability()
    return f"{major}.{minor}"


def is_sm90() -> bool:
    return get_compute_version() == "9.0"


def is_sm100() -> bool:
    return get_compute_version().startswith("10.")


def is_sm12x() -> bool:
    return get_compute_version().startswith("12.")
