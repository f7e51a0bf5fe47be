"""CPU oracle for the foveated hot path (sensor grid-sample + KNNConv).

TEST INFRASTRUCTURE ONLY.  Nothing under this directory is part of the shipped
product: only the test-suite, the smoke check and the benchmark's CPU-baseline
leg may import it, and only as the checker that CUDA results are compared with.

Parity status: PINNED.  The functions here are checked (bit-exact for the
sampler, 1e-5 relative for KNNConv in fp32) against outputs of the reference's
own PyTorch CPU implementation; those outputs are committed as fixtures under
``tests/golden/`` together with the script that produced them
(``tests/golden/make_golden.py``).
"""
from .fovi_oracle import *  # noqa: F401,F403
