"""CPU oracle for the compact-DMS decode path.  TEST INFRASTRUCTURE ONLY.

This package restates, in plain numpy, the algorithms of the reference project's compact-DMS
decode path (file:line citations are on every function).  It exists so that the CUDA kernels can
be checked against an independent implementation; nothing in the shipped package
(`fastdms_b200/`) imports it.  Only the test-suite, the smoke check and the CPU-baseline leg of
the benchmark may call into it.

Parity status: PINNED.  `tests/test_oracle_golden.py` checks every function here against
`tests/golden/ops_golden.npz`, which was produced by running the reference's own CPU code paths
(`tests/golden/make_golden_ops.py`), and against the known-answer vectors of the reference's
unit tests (pack offsets/counts/positions, decode metadata, decision recording, threshold +-1 ulp,
expiry with capacity 9 / window 3).

Conventions
-----------
* Float tensors are passed as float32 numpy arrays holding already-rounded values (a bf16 tensor
  is the float32 array of its exact values).  `dtypes.round_to(x, "bf16")` performs the rounding.
* FP8 e4m3 tensors are passed as raw bytes (uint8); `e4m3.decode` / `e4m3.encode` convert.
* Integer/bool metadata uses int32 / bool arrays with the reference's shapes.
"""
