"""Measurement drivers, not part of the backend: they launch the library's kernels through the C ABI on the
benchmark configurations' shapes so that CUDA events and ncu can time them (the commands quoted in
profiles/ run these).  Nothing in the backend imports this package."""
