"""Shared pytest configuration: the ``gpu`` marker and small helpers."""

from __future__ import annotations

import pathlib
import sys

import pytest
import torch

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100a) GPU")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def load_golden(name: str):
    return torch.load(GOLDEN / f"{name}.pt", weights_only=True)


def rebuild_cache(case, which: str, device="cpu"):
    """Dense cache tensor from the sparse form stored in the RoPE fixture."""
    dtype = case[f"{which}_values"].dtype
    cache = torch.full(case["cache_shape"], -999.0, dtype=dtype)
    cache.view(-1)[case[f"{which}_index"]] = case[f"{which}_values"]
    return cache.to(device)


def ordered_bits(t: torch.Tensor) -> torch.Tensor:
    """Map 16-bit float patterns to integers that are monotonic in value, so
    that |a - b| counts representable values between two numbers (ulps)."""
    bits = t.contiguous().view(torch.int16).to(torch.int32)
    return torch.where(bits < 0, -(bits & 0x7FFF), bits)


def ulp_distance16(a: torch.Tensor, b: torch.Tensor) -> int:
    return int((ordered_bits(a) - ordered_bits(b)).abs().max())


def rel_l2(actual: torch.Tensor, expected: torch.Tensor) -> float:
    diff = actual.double() - expected.double()
    return float(diff.norm() / expected.double().norm().clamp_min(1e-12))
