"""CPU restatement of the reference algorithms — TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory.  It exists so that the CUDA
kernels can be checked against an independent, slow, obviously-correct statement of
what the reference computes (``tests/``, the smoke check and the CPU leg of the
benchmark are its only users).  Every function cites the reference lines it restates.
Parity is pinned: ``tests/test_oracle_golden.py`` checks these functions against
fixtures produced by running the reference itself (``tests/golden/generate.py``).
"""
