"""Sparse-format bit flags (python/gs/format.py:1-3 in gSampler)."""
_CSR = 4
_CSC = 2
_COO = 1
