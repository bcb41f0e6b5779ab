"""CPU oracle for the SAM image-encoder path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; only the test-suite, the smoke check and the benchmark's CPU
baseline leg call into it, and only as the checker / reported baseline.
"""
