"""CPU oracle for the fused RMSNorm -> Linear path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory: only the test-suite, the smoke check and the CPU-baseline leg of
the benchmark may, and there only as the checker / the timed CPU baseline.
"""
