"""Test infrastructure only: CPU checkers for the attention kernels (never imported by the product path)."""
