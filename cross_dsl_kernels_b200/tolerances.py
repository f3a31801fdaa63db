"""Pass/fail thresholds for the FP32 projection, as upstream defines them in
src/crossdsl_kernels/tolerances.py:7-25: an absolute bound that grows with
sqrt(K) past K=1024 and a fixed relative-L2 bound."""

from __future__ import annotations

import math
from typing import Any

_ABS_BASE = 2.0e-4
_REL_L2 = 1.0e-5


def fp32_gemv_tolerance(k: int) -> dict[str, Any]:
    if k <= 0:
        raise ValueError("k must be positive")
    return {
        "dtype": "float32",
        "max_abs_err": _ABS_BASE * max(1.0, math.sqrt(k / 1024.0)),
        "rel_l2_err": _REL_L2,
        "k": k,
        "policy": "max_abs_err <= 2e-4 * max(1, sqrt(K / 1024)) and rel_l2_err <= 1e-5",
        "max_rel_err_role": "diagnostic-only; near-zero reference values can dominate elementwise relative error",
    }


def fp32_gemv_status(k: int, max_abs_err: float, rel_l2_err: float) -> tuple[str, dict[str, Any]]:
    limits = fp32_gemv_tolerance(k)
    ok = max_abs_err <= limits["max_abs_err"] and rel_l2_err <= limits["rel_l2_err"]
    return ("PASS" if ok else "FAIL"), limits
