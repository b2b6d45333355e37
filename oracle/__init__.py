"""CPU oracle for the gpt-oss attention path: test infrastructure, never shipped code.

Only the tests, the smoke check and the benchmark's CPU-baseline leg import this.
"""
