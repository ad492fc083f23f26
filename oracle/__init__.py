"""CPU oracles for the streaming-attention path (TEST INFRASTRUCTURE ONLY).

Nothing under ``oracle/`` is part of the shipped product: only the tests, the
smoke check and the CPU-baseline leg of the benchmark may import it, and only
as the checker.  The product (``kernels_b200``) never imports this package.
"""
