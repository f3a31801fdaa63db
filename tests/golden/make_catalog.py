"""Writes tests/golden/shape_catalog.json from an upstream checkout's own shape catalogs.

    python tests/golden/make_catalog.py /path/to/cross_dsl_kernels

The fixture lists, by upstream's case names, the shapes upstream benchmarks and verifies: the 25 FP32 cases of
benchmarks/shapes/comparison.json and the 16 W4A16 cases of benchmarks/shapes/w4a16.json (tails included), plus the
base seed of benchmarks/compare.py (case i is drawn from seed + i).  tests/test_gpu_catalog.py runs every one of them
through this library's kernels.
"""

from __future__ import annotations

import json
import pathlib
import re
import sys


def main() -> int:
    if len(sys.argv) != 2:
        print(__doc__, file=sys.stderr)
        return 2
    checkout = pathlib.Path(sys.argv[1])
    shapes = checkout / "benchmarks" / "shapes"
    fp32 = json.loads((shapes / "comparison.json").read_text())["cases"]
    w4 = json.loads((shapes / "w4a16.json").read_text())["cases"]
    seed = int(re.search(r'"--seed", type=int, default=(\d+)', (checkout / "benchmarks" / "compare.py").read_text()).group(1))
    out = {"source": "benchmarks/shapes/comparison.json, benchmarks/shapes/w4a16.json, benchmarks/compare.py (--seed default)",
           "base_seed": seed, "fp32": fp32, "w4a16": w4}
    target = pathlib.Path(__file__).resolve().parent / "shape_catalog.json"
    target.write_text(json.dumps(out, indent=1) + "\n")
    print(f"{target}: {len(fp32)} FP32 cases, {len(w4)} W4A16 cases, base seed {seed}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
