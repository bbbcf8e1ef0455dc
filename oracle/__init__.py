"""CPU oracle for the speculative-decoding hot path.

TEST INFRASTRUCTURE ONLY.  This package is a NumPy restatement of the
reference algorithm (VerseNext `verse_nex` / `verse_torch`, fp32 CPU path).
It exists to check the CUDA library and to time a CPU baseline.  Nothing in
`versenext_b200/` imports it; only `tests/`, `__graft_entry__.smoke()` and the
CPU-baseline / reference legs of `bench.py` may.

Parity status
-------------
* Greedy path (draft -> verify -> accept-longest-prefix) and the target model
  forward are PINNED: `tests/golden/make_golden.py` ran the real reference
  classes and committed their outputs; `tests/test_oracle.py` checks this
  restatement against those fixtures.
* Rejection sampling, residual sampling, Philox uniforms, tree verification,
  bonus token, KV commit/rollback, group-128 INT4 and bf16 rounding have no
  counterpart in the reference: for those this oracle is a restatement of the
  published algorithms composed from reference primitives (softmax /
  temperature / top-k semantics, model forward) and is "parity unpinned".
"""

from . import philox, accept, model, quant, spec  # noqa: F401
