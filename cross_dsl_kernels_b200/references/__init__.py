"""Host-side helpers that keep upstream's ``crossdsl_kernels.references`` names.

Only the integer address helpers and the set-up validator live here; the
floating-point reference implementations of the ops are not part of this
library (its ops run on the GPU or raise).
"""

from .paged_address import PagedAddress, address_for_token, hnd_linear_index, nhd_linear_index
from .rope_kv import validate_paged_kv_indices

__all__ = [
    "PagedAddress",
    "address_for_token",
    "hnd_linear_index",
    "nhd_linear_index",
    "validate_paged_kv_indices",
]
