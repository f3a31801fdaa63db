"""Set-up validation for the RoPE + paged K/V append op.

The device kernel trusts its index tensors (as upstream's kernels do); callers
establish that trust once, at set-up, with :func:`validate_paged_kv_indices`,
which keeps the name, keywords and error behaviour of upstream's
src/crossdsl_kernels/references/rope_kv.py:73-103.
"""

from __future__ import annotations

from typing import Any

from .paged_address import address_for_token


def validate_paged_kv_indices(positions: Any, page_table: Any, sequence_ids: Any, *,
                              page_size: int, num_cache_pages: int, max_position: int) -> None:
    """Raise ValueError unless every token's indices are in range and no two
    tokens map to the same (physical page, offset) slot.

    Reads the index tensors on the host, so it synchronises when they live on
    a GPU: call it when the batch is built, not per decode step.
    """
    if page_size <= 0:
        raise ValueError("page_size must be positive")
    if positions.dim() != 1 or sequence_ids.shape != positions.shape:
        raise ValueError("positions and sequence_ids must be matching vectors")
    if page_table.dim() != 2:
        raise ValueError("page_table must be shaped [sequences, logical_pages]")
    rows = page_table.cpu().tolist()
    seen = set()
    for pos, seq in zip(positions.cpu().tolist(), sequence_ids.cpu().tolist()):
        if seq < 0 or seq >= len(rows):
            raise ValueError("sequence ID is out of bounds")
        if pos < 0 or pos >= max_position:
            raise ValueError("position is outside the trigonometric table")
        where = address_for_token(pos, page_size, rows[seq])
        if where.physical_page >= num_cache_pages:
            raise ValueError("physical page ID is outside the cache")
        slot = where.physical_page * page_size + where.offset
        if slot in seen:
            raise ValueError("tokens must write distinct physical cache slots")
        seen.add(slot)
