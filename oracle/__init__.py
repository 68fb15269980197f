"""CPU oracle for the TCFP-12 linear-layer hot path.

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this
directory; only the test-suite, the smoke check and the CPU-baseline leg of
the benchmark may call into it, and only as the checker / the thing timed as
"the reference's CPU path" -- never as a fallback for the CUDA kernels.
"""
