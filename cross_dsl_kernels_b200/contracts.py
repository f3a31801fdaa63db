"""Metadata-only storage checks shared by the op frontends
(upstream: src/crossdsl_kernels/contracts.py:30-44)."""

from __future__ import annotations

from typing import Any, Iterable


def _byte_span(t: Any) -> tuple[int, int]:
    """[first byte, one past the last byte) that the tensor's elements can touch.  For a contiguous tensor this
    is numel * element_size from data_ptr(); for a strided view (a column slice of a wider matrix) the last
    element sits at sum((size - 1) * stride) elements from data_ptr(), so the span is wider than numel."""
    start = t.data_ptr()
    if t.numel() == 0:
        return start, start
    reach = sum((size - 1) * stride for size, stride in zip(t.shape, t.stride()))
    return start, start + (reach + 1) * t.element_size()


def storage_overlaps(a: Any, b: Any) -> bool:
    """True when the byte spans of two tensors (contiguous or positively strided) intersect."""
    if a.numel() == 0 or b.numel() == 0:
        return False
    a0, a1 = _byte_span(a)
    b0, b1 = _byte_span(b)
    return a0 < b1 and b0 < a1


def validate_cache_storage(inputs: Iterable[Any], k_cache: Any, v_cache: Any) -> None:
    """The append op writes both caches while it reads its inputs, so neither
    cache may alias the other or any input.  Spans are exact for contiguous
    tensors and conservative for strided views such as q/k/v slices of a fused
    QKV matrix (the gaps between their rows count as theirs)."""
    if storage_overlaps(k_cache, v_cache) or any(
        storage_overlaps(cache, t) for cache in (k_cache, v_cache) for t in inputs
    ):
        raise ValueError("KV caches must not overlap each other or the input tensors")
