"""CPU oracle for the AUSSM selective-scan path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this directory: it is the checker
that the parity tests, the smoke check and the CPU-baseline leg of the
benchmark use.  Every function restates, in plain PyTorch on the CPU, an
algorithm of the reference project and cites the reference lines it follows.

Parity status: pinned.  The restatements are compared against outputs of the
reference's own Python oracles (imported from the reference checkout by
``tests/golden/make_golden.py``) that are stored under ``tests/golden``.
"""
