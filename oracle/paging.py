"""Integer address arithmetic of the paged K/V cache (oracle side).

Follows src/crossdsl_kernels/references/paged_address.py:14-56 of the upstream
project: a token position is split into a logical page and an in-page offset,
the logical page is looked up in the sequence's page-table row, and the
resulting (physical page, offset, head, dim) tuple is flattened for one of two
cache layouts.  numpy int64 throughout so that whole batches translate at once.
"""

from __future__ import annotations

import numpy as np


def translate(positions, sequence_ids, page_table, page_size: int):
    """Vectorised page walk: returns (physical_page, offset) int64 arrays.

    Mirrors address_for_token (paged_address.py:14-29), including its three
    rejections (non-positive page size, negative position, negative physical
    page -> ValueError) and the out-of-table lookup (-> IndexError).
    """
    if page_size <= 0:
        raise ValueError("page_size must be positive")
    pos = np.asarray(positions, dtype=np.int64)
    seq = np.asarray(sequence_ids, dtype=np.int64)
    table = np.asarray(page_table, dtype=np.int64)
    if (pos < 0).any():
        raise ValueError("position must be non-negative")
    logical = pos // page_size
    if (logical >= table.shape[1]).any():
        raise IndexError("position requires a page beyond the page table row")
    physical = table[seq, logical]
    if (physical < 0).any():
        raise ValueError("physical page IDs must be non-negative")
    return physical, pos % page_size


def flat_index(layout: str, page, offset, head, dim, *, page_size: int, num_heads: int, head_dim: int):
    """Element index into a contiguous cache.

    NHD is cache[page, offset, head, dim] (paged_address.py:32-43),
    HND is cache[page, head, offset, dim] (paged_address.py:46-56).
    """
    if layout == "NHD":
        return ((page * page_size + offset) * num_heads + head) * head_dim + dim
    if layout == "HND":
        return ((page * num_heads + head) * page_size + offset) * head_dim + dim
    raise ValueError("layout must be NHD or HND")
