"""CPU oracle for stick-breaking attention.  TEST INFRASTRUCTURE ONLY.

Nothing in the product package imports this directory; only the test-suite, the
smoke check and the CPU-baseline leg of the benchmark may use it.
"""
