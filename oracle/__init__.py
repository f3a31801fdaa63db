"""CPU oracle for the four decode ops: TEST INFRASTRUCTURE, not product code.

This package restates, op by op, the arithmetic of the upstream PyTorch
references (paths are relative to the upstream project):

* src/crossdsl_kernels/references/rmsnorm.py   -> :func:`oracle.decode_ops.residual_rmsnorm`
* src/crossdsl_kernels/references/gemv.py      -> :func:`oracle.decode_ops.decode_projection`
* src/crossdsl_kernels/references/rope_kv.py   -> :func:`oracle.decode_ops.rope_paged_append`
* src/crossdsl_kernels/references/paged_address.py -> :mod:`oracle.paging`
* src/crossdsl_kernels/quantization.py         -> :mod:`oracle.int4`

Only the test-suite, the smoke check and the benchmark's CPU-baseline leg may
import it.  The shipped library (``cross_dsl_kernels_b200``) never does: its
ops run on the GPU or raise.

Parity pin: every function here is checked bit-for-bit against outputs of the
upstream Python functions on seeded inputs (fixtures under ``tests/golden``,
written by ``tests/golden/make_golden.py``) and against the known-answer
vectors that upstream's own unit tests hold.
"""
