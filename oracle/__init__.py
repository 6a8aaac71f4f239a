"""CPU oracle for the quantised-linear hot path — TEST INFRASTRUCTURE ONLY.

Plain numpy / CPU-torch restatements of the anima-trainer algorithms that the
CUDA library implements; every function cites the reference file:line it follows.
Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this package, and only as the checker: the product
(``anima_trainer_sm120_b200`` and ``libanima_b200.so``) never does.

Parity pin: the restatements are checked against golden vectors produced by the
reference's own code — its Triton kernels run under the Triton CPU interpreter
and its CPU-capable torch paths imported unmodified (``tests/golden/make_golden.py``
made them; ``tests/test_oracle_golden.py`` checks them).
"""
