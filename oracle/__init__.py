"""CPU oracle for the packed-KV hot path (TEST INFRASTRUCTURE, not product code).

Everything in this package is a plain-numpy restatement of the reference
algorithms (quantise + bit-pack, Lagrangian bit allocation, dequantise-then-
attend).  It exists only so that the tests, the smoke check and the CPU
baseline leg of the benchmark have something independent to compare the CUDA
path with.  Nothing in ``rdkv_b200`` may import it.

Parity status: pinned.  ``tests/golden/make_golden.py`` runs the reference's
own Python code on seeded inputs and stores its outputs; ``tests/
test_oracle_golden.py`` checks this oracle bit-for-bit against those files.
"""
