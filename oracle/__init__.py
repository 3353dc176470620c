"""CPU oracle for the pi0 hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory.  It is used by the
tests, by the smoke check and by the CPU-baseline leg of the benchmark as the
checker; it is never the thing that is measured as the product or shipped.
"""
