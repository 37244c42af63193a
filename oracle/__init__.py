"""CPU oracle: numpy restatements of the reference's algorithms for the hot path.

TEST INFRASTRUCTURE ONLY. Nothing under this directory is part of the product: it is imported
only by tests/, by __graft_entry__.smoke() as the checker, and by bench.py's cpu_baseline /
``--impl reference`` legs as the thing timed on host cores. The product path (the package next to
this directory) never imports it and has no CPU fallback.

Parity pinning: every function here is checked in tests/test_oracle_golden.py against vectors
produced by the reference's own code (tests/golden/make_golden.py imports the reference's
numpy oracles and structured-pattern generators and stores their inputs and outputs), and against
the known-answer cases of the reference's test-suite. The mixed prefill/decode restatement has no
reference oracle and no reference test: for that function alone, parity is unpinned.
"""
