"""Tensor-level operators of the B200 backend (thin wrappers over the C ABI)."""
