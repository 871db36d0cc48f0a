"""Optional operator sets built on the same kernels."""
