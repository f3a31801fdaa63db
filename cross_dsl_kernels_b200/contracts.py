"""Metadata-only storage checks shared by the op frontends
(upstream: src/crossdsl_kernels/contracts.py:30-44)."""

from __future__ import annotations

from typing import Any, Iterable


def _byte_span(t: Any) -> tuple[int, int]:
    start = t.data_ptr()
    return start, start + t.numel() * t.element_size()


def storage_overlaps(a: Any, b: Any) -> bool:
    """True when two contiguous tensors share at least one byte."""
    if a.numel() == 0 or b.numel() == 0:
        return False
    a0, a1 = _byte_span(a)
    b0, b1 = _byte_span(b)
    return a0 < b1 and b0 < a1


def validate_cache_storage(inputs: Iterable[Any], k_cache: Any, v_cache: Any) -> None:
    """The append op writes both caches while it reads its inputs, so neither
    cache may alias the other or any input (all tensors are contiguous, hence
    byte intervals are exact)."""
    if storage_overlaps(k_cache, v_cache) or any(
        storage_overlaps(cache, t) for cache in (k_cache, v_cache) for t in inputs
    ):
        raise ValueError("KV caches must not overlap each other or the input tensors")
