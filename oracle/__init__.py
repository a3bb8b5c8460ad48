"""CPU oracle for the MSDA path. TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this package; the product path never does.
"""
