"""Checkers for the tests and the benchmark's CPU-baseline leg; not part of the product."""
