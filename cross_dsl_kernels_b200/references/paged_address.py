"""Paged K/V cache addressing: same names, arguments and errors as upstream's
src/crossdsl_kernels/references/paged_address.py:7-56.

The append kernel computes exactly these integers on the device
(csrc/rope_kv.cu); these host functions are what callers use to locate a
token's slot when they read the cache back.
"""

from __future__ import annotations

from typing import NamedTuple, Sequence


class PagedAddress(NamedTuple):
    """Where one token lives: its logical page within the sequence, its offset
    inside that page, and the physical cache page the table maps it to."""

    logical_page: int
    offset: int
    physical_page: int


def address_for_token(position: int, page_size: int, page_table_row: Sequence[int]) -> PagedAddress:
    """Walk one sequence's page-table row for ``position``.

    ValueError for a non-positive page size, a negative position or a negative
    physical page; IndexError when the row has no entry for the logical page.
    """
    if page_size <= 0:
        raise ValueError("page_size must be positive")
    if position < 0:
        raise ValueError("position must be non-negative")
    logical, offset = divmod(position, page_size)
    if logical >= len(page_table_row):
        raise IndexError("position requires a page beyond page_table_row")
    physical = int(page_table_row[logical])
    if physical < 0:
        raise ValueError("physical page IDs must be non-negative")
    return PagedAddress(logical, offset, physical)


def nhd_linear_index(physical_page: int, offset: int, head: int, dim: int, *,
                     page_size: int, num_heads: int, head_dim: int) -> int:
    """Element index of cache[page, offset, head, dim] (token-major pages)."""
    slot = physical_page * page_size + offset
    return (slot * num_heads + head) * head_dim + dim


def hnd_linear_index(physical_page: int, offset: int, head: int, dim: int, *,
                     page_size: int, num_heads: int, head_dim: int) -> int:
    """Element index of cache[page, head, offset, dim] (head-major pages)."""
    plane = physical_page * num_heads + head
    return (plane * page_size + offset) * head_dim + dim
