"""Measurement helpers that are not on the product path (the reference's kernels as a timing and parity anchor)."""
